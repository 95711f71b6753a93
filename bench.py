"""Benchmark of the MXFP4 quantized-linear path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload ("llama7b_linears_16384tok"): the four linear layers of a 7B Llama block
(QKV 4096->12288, O 4096->4096, gate/up 4096->22016, down 11008->4096), forward + dgrad + wgrad,
16384 tokens per GPU, bf16 activations ~N(0,1), fp32 master weights ~N(0,0.02), bf16 grad-outputs
~N(0,1e-3); synthetic, seeded.  One step = all layers once, through
quartet_b200.quantization.QuantizedLinear (forward + backward).  Token rows are sharded over the
GPUs (weak scaling: the same number of tokens on every GPU); the per-GPU weight-gradient partials are
averaged inside the step, every rank ending up with its row shard (--exchange: rows pushed into their
owner's memory by the DMA engines or by the GEMM's own stores, or an NCCL reduce-scatter).
Metric: model FLOP/s = 6*M*N*K per layer, summed over layers and GPUs.

Secondary workloads (same code path, their own JSON line): "quantized_linear_8192x640x2560" (one
layer, X [8192, 640], W [2560, 640]), "llama30m_linears_32768tok" (the 24 block linears of the
30M model, d 640, SwiGLU 1792, at batch 64 x 512 tokens), "llama3_8b_linears_32768tok" (the four
block linears of a Llama-3-8B layer at 8 x 4096 tokens), and "llama30m_step": a whole training step
(forward, backward under bf16 autocast, AdamW) of a 30M Llama-style model whose block linears are
QuantizedLinear (6 blocks, width 640, 5 heads, SwiGLU 1792, vocabulary 32000, 64 x 512 uniform-random
token ids; the model is the test harness tests/llama_harness.py; add --compile for torch.compile and
--fuse-producers for the norms and the SwiGLU product computed inside the forward quantizers).

What the line reports:
  value      K steps with inputs resident in HBM, CUDA events, max over ranks
  e2e        the same through host buffers: every step copies each layer's activations and
             grad-outputs from pinned host memory and copies y, dx and this rank's dW shard back into
             pinned host memory, all inside the timed region
  roofline   the GEMM kernel, timed per launch with CUDA events in a short pass (a burst: compared
             with 4 x the measured bf16 burst rate) and again in a pass of several seconds (compared
             with 4 x the measured sustained rate), plus the fraction of the nominal 9 PFLOP/s
  sustained  the step looped for >= 3 s in one timed region, with the SM clock sampled meanwhile
  boundary_exceptions  forward-quantizer codes / scale bytes / mask bits of a row sample of the
             bench inputs compared with the CPU oracle (the oracle is the checker here)

`--impl reference` times the reference's own pseudo-quantized arithmetic for the same layers on the
host CPU (the torch-fp32 restatement in oracle/ref_math.py, which is pinned bit-exactly to the
reference kernel) on a bounded token sample.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "llama7b_linears_16384tok": {"tokens": 16384, "layers": [("qkv", 4096, 12288), ("o", 4096, 4096), ("gate_up", 4096, 22016), ("down", 11008, 4096)]},
    "quantized_linear_8192x640x2560": {"tokens": 8192, "layers": [("fc", 640, 2560)]},
    # the block linears of a Llama-3-8B layer (32 query / 8 key-value heads of 128: fused QKV is 4096 -> 6144; SwiGLU 14336) at 8 x 4096 tokens
    "llama3_8b_linears_32768tok": {"tokens": 32768, "layers": [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672), ("down", 14336, 4096)]},
    "llama30m_linears_32768tok": {"tokens": 32768, "layers": [(f"{name}{i}", k, n) for i in range(6) for name, k, n in
                                                               (("c_attn", 640, 1920), ("attn_proj", 640, 640), ("w12", 640, 3584), ("c_proj", 1792, 640))]},
}
WORKLOAD = "llama7b_linears_16384tok"
LAYERS = WORKLOADS[WORKLOAD]["layers"]
TOKENS = WORKLOADS[WORKLOAD]["tokens"]
CPU_SAMPLE_TOKENS = int(os.environ.get("QUARTET_BENCH_CPU_TOKENS", "512"))  # token sample of the CPU arm (the tests shrink it)
METRIC = "quantized_linear_fwd_bwd_tflops"
NOMINAL_MXFP4_TFLOPS = 9000.0  # dense MXFP4 of one B200, vendor figure
SUSTAINED_SECONDS = float(os.environ.get("QUARTET_BENCH_SUSTAINED_S", "3.0"))


def gemm_algorithmic_bytes(m, n, k, out_bytes):
    return (m + n) * k * (0.5 + 1.0 / 32.0) + m * n * out_bytes


def read_ncu_summary(path):
    """Metric rows of a tracked ncu summary (profiles/*.md): {metric: first-launch value}, sizes in bytes.
    Returns {} when the file does not exist."""
    out = {}
    try:
        text = open(path).read()
    except OSError:
        return out
    unit_scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    for line in text.splitlines():
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) >= 3 and re.fullmatch(r"[a-z0-9_.]+", cells[0] or "-"):
            try:
                out[cells[0]] = float(cells[2]) * unit_scale.get(cells[1], 1.0)
            except ValueError:
                pass
    m = re.search(r"--m (\d+) --n (\d+) --k (\d+)", text)
    if m:
        out["shape"] = tuple(int(v) for v in m.groups())
    return out


def gemm_traffic_per_launch(layers, tokens, capture):
    """DRAM bytes of the step's average GEMM launch: the captured launch's traffic scaled by algorithmic bytes
    (operands + scales + result).  (traffic, algorithmic) or (None, algorithmic) without a capture."""
    alg = 0.0
    for _, k, n in layers:
        alg += gemm_algorithmic_bytes(tokens, n, k, 2) + gemm_algorithmic_bytes(tokens, k, n, 2) + gemm_algorithmic_bytes(n, k, tokens, 4)
    alg /= 3 * len(layers)
    if not capture or "shape" not in capture or "dram__bytes_read.sum" not in capture:
        return None, alg
    m, n, k = capture["shape"]
    ratio = (capture["dram__bytes_read.sum"] + capture["dram__bytes_write.sum"]) / gemm_algorithmic_bytes(m, n, k, 2)
    return ratio * alg, alg


def layer_flops(m, layers=None):
    return sum(6.0 * m * k * n for _, k, n in (layers or LAYERS))


def load_peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return {"hbm": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "note": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "note": "fallback"}


def bench_config(workload, world, exchange):
    w = WORKLOADS[workload]
    par = f"dp{world} token-row shards"
    if world > 1:
        par += {"peer": " + wgrad rows stored to their owner by the GEMM (peer memory)", "copy": " + wgrad rows pushed to their owner by the DMA engines",
                "nccl": " + NCCL reduce-scatter of wgrad", "auto": " + wgrad rows pushed to their owner by the DMA engines"}[exchange]
    return {"workload": workload, "tokens_per_gpu": w["tokens"], "layers": [[n_, k, n] for n_, k, n in w["layers"]],
            "activations": "bf16", "weights": "fp32 master", "parallelism": par,
            "l2": "inputs larger than L2 (126 MB): every step streams its operands from HBM"}


# ----------------------------------------------------------------------------------------------
# CPU arm (the reference's arithmetic on host cores)
# ----------------------------------------------------------------------------------------------
def cpu_arm(steps, warmup, layers, tokens_full, tokens=None):
    import torch

    from oracle import ref_math as rm

    tokens = min(tokens or CPU_SAMPLE_TOKENS, tokens_full)
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(0)
    data = []
    for _, k, n in layers:
        x = torch.randn(tokens, k, generator=gen).bfloat16().float()
        w = (torch.randn(n, k, generator=gen) * 0.02).bfloat16().float()
        e = (torch.randn(tokens, n, generator=gen) * 1e-3).bfloat16().float()
        data.append((x, w, e))
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for x, w, e in data:
            rm.cpu_layer_fwd_bwd(x, w, e, seed=it)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    dt = sum(times) / len(times)
    return layer_flops(tokens, layers) / dt / 1e12, dt, cores, f"{tokens} of {tokens_full} tokens per layer, all {len(layers)} layers, fp32 torch ops"


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) every few ms."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index, period_s=0.004):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.stop_flag, self.thread, self.max_mhz, self.err = threading.Event(), None, None, None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # noqa: BLE001
            self.err = f"nvml unavailable: {e}"
            return self
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def _run(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception as e:  # noqa: BLE001
                self.err = str(e)
                return
            time.sleep(self.period)

    def stop(self):
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.err or "not sampled"]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        sm = sorted(self.samples)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# parity of a row sample of the bench inputs with the oracle
# ----------------------------------------------------------------------------------------------
def boundary_exceptions(ops, samples):
    """Forward-quantizer output of `samples` (device tensors [rows, cols]) against the CPU oracle: how many
    scale bytes, codes (outside groups whose scale differs) and mask bits differ, and how many elements sit
    exactly on a rounding tie in the oracle's arithmetic (those round toward the smaller magnitude in both)."""
    import torch

    from oracle import ref_math as rm

    tot = {"elements": 0, "scale_groups": 0, "codes": 0, "mask_bits": 0, "exact_ties": 0}
    for x in samples:
        rows, cols = x.shape
        h = rm.hadamard32(x.dtype)
        xc = x.detach().float().cpu()
        ref = rm.quant_fwd(xc, h)
        codes, sf, mask = ops.quant_fwd(x.detach().contiguous(), float(h[0, 0]), ops.QUEST_GAUSSIAN_SCALE)
        c = codes.cpu()
        full = torch.stack([c & 0xF, c >> 4], dim=-1).reshape(rows, cols).to(torch.int32)
        idx, neg = full & 7, (full & 8) != 0
        e8 = rm.from_blocked(sf.cpu(), rows, cols // 32)
        sf_bad = e8 != ref.e8m0
        grp = sf_bad.repeat_interleave(32, dim=1)
        code_bad = ((idx != ref.idx) | ((neg != ref.neg) & (idx != 0) & (ref.idx != 0))) & ~grp
        bits = torch.arange(8, dtype=torch.uint8)
        mk = ((mask.cpu().unsqueeze(-1) >> bits) & 1).bool().reshape(rows, cols)
        v = (rm.rotate(xc, h) / ref.shared.reshape(-1, 1)).abs()
        ties = sum(int((v == t).sum()) for t in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0))
        tot["elements"] += rows * cols
        tot["scale_groups"] += int(sf_bad.sum())
        tot["codes"] += int(code_bad.sum())
        tot["mask_bits"] += int(((mk != ref.mask) & ~grp).sum())
        tot["exact_ties"] += ties
    tot["note"] = "forward quantizer vs the CPU oracle on the first 256 rows of every layer's activations and weights"
    return tot


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def gpu_arm(args):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    layers_spec, tokens = WORKLOADS[args.workload]["layers"], WORKLOADS[args.workload]["tokens"]
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"  # the version banner goes to stdout, which carries the one JSON line
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if rank == 0:
        entry.build()
    if world > 1:
        dist.barrier()
    from quartet_b200 import ops
    from quartet_b200.quantization import BACKWARD_SCHEMES, QUANTIZER_CLASSES, QuantizedLinear
    from quartet_b200.shard import PeerSetupError, PeerWgradScatter, WgradReduceScatter
    from quartet_b200.staging import HostDrain, HostStager

    # ---- model + data (seeded; weights identical on every rank, activations differ per rank) ----
    gw = torch.Generator(device="cpu").manual_seed(0)
    layers, xs, es, xs_host, es_host = [], [], [], [], []
    for _, k, n in layers_spec:
        lin = QuantizedLinear(
            k, n, bias=False,
            weight_quantizer=QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
            activation_quantizer=QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
            gradient_quantizer=QUANTIZER_CLASSES["AlbertTsengQuantizer"](stochastic=True, rerotate="signs"),
            backward_scheme=BACKWARD_SCHEMES["Q(E)Q(Wt)t_Q(Et)Q(Xt)t"](),
        )
        with torch.no_grad():
            lin.weight.copy_(torch.randn(n, k, generator=gw) * 0.02)
        layers.append(lin.to(dev))
    torch.manual_seed(1000 + rank)
    for _, k, n in layers_spec:
        xh = torch.randn(tokens, k, dtype=torch.bfloat16).pin_memory()
        eh = (torch.randn(tokens, n) * 1e-3).to(torch.bfloat16).pin_memory()
        xs_host.append(xh), es_host.append(eh)
        xs.append(xh.to(dev).requires_grad_(True)), es.append(eh.to(dev))
    # pinned host buffers the end-to-end leg copies each step's results into: y, dx, this rank's rows of dW
    shard_ok = all(n % world == 0 for _, _, n in layers_spec)
    out_host = [(torch.empty(tokens, n, dtype=torch.bfloat16).pin_memory(), torch.empty(tokens, k, dtype=torch.bfloat16).pin_memory(),
                 torch.empty(n // world if shard_ok else n, k, dtype=torch.float32).pin_memory()) for _, k, n in layers_spec]
    # wgrad exchange across ranks
    reducer = sink = None
    if args.exchange == "auto":
        # measured on 2 and on 8 GPUs: the DMA-engine push costs less than the slowdown of a GEMM whose epilogue
        # stores cross NVLink
        args.exchange = "copy"
    if world > 1 and args.exchange in ("peer", "copy"):
        sink = PeerWgradScatter(device=dev, transport="store" if args.exchange == "peer" else "copy")
        try:
            for lin in layers:
                sink.prepare(lin.weight)
            for lin in layers:
                lin.wgrad_sink = sink
        except (PeerSetupError, ValueError) as exc:  # raised on every rank alike: fall back to the library collective everywhere
            if rank == 0:
                print(f"bench: {exc}; using the NCCL reduce-scatter", file=sys.stderr)
            sink.close()  # collective: frees the receive buffers of the layers prepared before the failing one
            sink, args.exchange = None, "nccl"
    if world > 1 and sink is None:
        reducer = WgradReduceScatter(world)

    # ---- count launches of this library's kernels and time them per kind ----
    counts = {"n": 0}
    timing = {"on": False, "rec": []}

    def wrap(name, fn, work):
        def inner(*a, **k):
            counts["n"] += 1
            if not timing["on"]:
                return fn(*a, **k)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn(*a, **k)
            e.record()
            timing["rec"].append((name, s, e, work(*a, **k)))
            return out

        return inner

    def q_bytes(per_elem, with_mask=0.0):
        return lambda x, *a, **k: ("bytes", x.numel() * (x.element_size() + per_elem + (with_mask if k.get("return_mask", True) else 0)))

    def gemm_work(a_, asf, b_, *r, **k):
        return ("flops", 2.0 * a_.shape[0] * b_.shape[0] * a_.shape[1] * 2)

    ops.quant_fwd = wrap("quant_fwd", ops.quant_fwd, q_bytes(0.53125, 0.125))
    ops.quant_bwd = wrap("quant_bwd", ops.quant_bwd, lambda x, *a, **k: ("bytes", x.numel() * (x.element_size() + 0.53125)))
    ops.quant_bwd_t = wrap("quant_bwd_t", ops.quant_bwd_t, lambda x, *a, **k: ("bytes", x.numel() * (x.element_size() + 0.53125)))
    ops.quant_bwd_dual = wrap("quant_bwd_dual", ops.quant_bwd_dual, lambda x, *a, **k: ("bytes", x.numel() * (x.element_size() + 2 * 0.53125)))
    ops.requant_t = wrap("requant_t", ops.requant_t, lambda c, *a, **k: ("bytes", c.numel() * 2 * 1.0625))
    ops.gemm_mxfp4_tn_scatter = wrap("gemm", ops.gemm_mxfp4_tn_scatter, gemm_work)
    ops.shard_reduce = wrap("shard_reduce", ops.shard_reduce, lambda ptr, n_slots, elems, *r, **k: ("bytes", (n_slots + 1) * elems * 4))
    ops.gemm_mxfp4_tn = wrap("gemm", ops.gemm_mxfp4_tn, gemm_work)
    # the layer's one-call entry points launch 3 (forward) and 5 (backward: dual quantizer, two re-quantizers, two GEMMs) kernels
    real_fwd, real_bwd = ops.linear_fwd, ops.linear_bwd

    def counted_fwd(*a, **k):
        counts["n"] += 3
        return real_fwd(*a, **k)

    def counted_bwd(*a, **k):
        counts["n"] += 5
        return real_bwd(*a, **k)

    ops.linear_fwd, ops.linear_bwd = counted_fwd, counted_bwd

    stager, drain = HostStager(dev), HostDrain(dev)
    for i in range(len(layers)):
        stager.register(i, (xs[i], es[i]))
    pending = {"items": 0}  # how many (step, layer) items of the current timed run are still to be prefetched
    deferred = {}           # the exchange join of the step before

    def prefetch_next(i):
        if pending["items"] > 0:
            pending["items"] -= 1
            stager.prefetch(i, (xs_host[i], es_host[i]))

    def step(from_host=False):
        for i, lin in enumerate(layers):
            if from_host:
                stager.acquire(i)                       # compute stream waits for this layer's inputs
                prefetch_next((i + 1) % len(layers))    # next layer's (or next step's first) inputs cross PCIe meanwhile
            xs[i].grad = None
            lin.weight.grad = None
            y = lin(xs[i])
            if i == 0:
                join_exchange()  # of the previous step: its last layer's exchange had this layer's forward to finish under
            y.backward(es[i])
            if reducer is not None:
                reducer.submit(lin.weight.grad)
            if from_host:
                drain.push(out_host[i][0], y.detach())  # results leave on their own stream while the next layer computes
                drain.push(out_host[i][1], xs[i].grad)
                stager.release(i)
                if world == 1:
                    drain.push(out_host[i][2], lin.weight.grad)
        if reducer is not None or sink is not None:
            # a step's exchange is joined after the first forward of the NEXT step (the last step's at the end of the
            # timed region): the last layer's rows cross NVLink under the next step's first kernels
            deferred["join"] = reducer.wait if reducer is not None else sink.wait
            deferred["to_host"] = from_host

    def join_exchange():
        fn = deferred.pop("join", None)
        if fn is None:
            return
        shards = fn()
        if deferred.pop("to_host", False):
            for i, dw in enumerate(shards):
                drain.push(out_host[i][2], dw)

    def timed(n_steps, from_host):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        if from_host:  # every (step, layer) item is copied exactly once, all inside the timed region
            pending["items"] = n_steps * len(layers)
            prefetch_next(0)
        for _ in range(n_steps):
            step(from_host)
        join_exchange()  # every step's exchange completes inside the region
        if from_host:
            drain.join()  # the region ends when the last result has reached host memory
        e.record()
        torch.cuda.synchronize()
        ms = torch.tensor([s.elapsed_time(e)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.barrier()
        return ms.item()

    def per_kernel(n_steps):
        """Per-launch CUDA-event timing of this library's kernels over n_steps steps."""
        timing["rec"] = []
        timing["on"] = True
        ops.FUSED_LAYER_CALLS = False  # entry points one by one, so that each launch can be bracketed by events
        for _ in range(n_steps):
            step()
        join_exchange()
        torch.cuda.synchronize()
        ops.FUSED_LAYER_CALLS = True
        timing["on"] = False
        agg = {}
        for name, s, e, (kind, work) in timing["rec"]:
            a = agg.setdefault(name, {"ms": 0.0, "work": 0.0, "kind": kind, "n": 0})
            a["ms"] += s.elapsed_time(e)
            a["work"] += work
            a["n"] += 1
        timing["rec"] = []
        return agg

    nvml_index = torch.cuda.current_device() if os.environ.get("CUDA_VISIBLE_DEVICES") is None else int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank])
    for _ in range(args.warmup):
        step()
    join_exchange()
    sampler = ClockSampler(nvml_index).start() if rank == 0 else None
    counts["n"] = 0
    total_ms = timed(args.steps, False)
    launches = counts["n"]
    clocks = sampler.stop() if rank == 0 else None

    timed(1, True)
    e2e_ms = timed(args.steps, True)

    agg = per_kernel(max(2, min(args.steps, 5)))
    # the same step for seconds on end (one timed region, no host synchronisation inside): clocks settle where
    # the power limit puts them.  The step count comes from the time measured above, identical on all ranks.
    sus_steps = max(args.steps, int(SUSTAINED_SECONDS * 1e3 / (total_ms / args.steps)) + 1)
    sampler = ClockSampler(nvml_index, 0.02).start() if rank == 0 else None
    sus_ms = timed(sus_steps, False)
    sus_clocks = sampler.stop() if rank == 0 else None
    agg_sus = per_kernel(sus_steps) if world == 1 else None

    exceptions = None
    if rank == 0:
        samples = [x[:256] for x in xs[:4]] + [lin.weight[:256] for lin in layers[:4]]
        exceptions = boundary_exceptions(ops, samples)
    status = ops.device_status()
    if sink is not None:
        sink.close()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = load_peaks()
    ms_per_step = total_ms / args.steps
    flops = layer_flops(tokens, layers_spec) * world
    value = flops / (ms_per_step * 1e-3) / 1e12

    def gemm_rate(a):
        g = a["gemm"]
        return g["work"] / (g["ms"] * 1e-3) / 1e12

    def quant_rate(a):
        qn = [k for k in a if k not in ("gemm", "shard_reduce")]
        q_ms = sum(a[k]["ms"] for k in qn)
        return sum(a[k]["work"] for k in qn) / (q_ms * 1e-3) / 1e9, qn

    gemm_tflops = gemm_rate(agg)
    q_gbs, qn = quant_rate(agg)
    burst_peak, sus_peak = 4 * peaks["bf16_burst"], 4 * peaks["bf16_sustained"]
    capture = read_ncu_summary(os.path.join(ROOT, "profiles", "gemm_mxfp4_2cta_8192x8192x4096.md"))
    traffic, alg = gemm_traffic_per_launch(layers_spec, tokens, capture)
    pipe = capture.get("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active")
    roofline = {
        "bound": "tensor", "kernel": "gemm_mxfp4_2cta_kernel", "achieved": round(gemm_tflops, 1), "peak": round(burst_peak, 1),
        "unit": "TFLOP/s", "frac": round(gemm_tflops / burst_peak, 4),
        "peak_note": f"4 x {peaks['note']} bf16 cuBLAS BURST rate ({peaks['bf16_burst']} TFLOP/s): the per-launch timing pass lasts well under a second. "
                     "4 x cuBLAS-bf16 is a stand-in for the MXFP4 peak (4:1 nominal ratio); the tensor-pipe counter of the ncu capture is the direct reading",
        "frac_of_nominal_9pf": round(gemm_tflops / NOMINAL_MXFP4_TFLOPS, 4),
        "ncu_tensor_pipe_active_pct": round(pipe, 1) if pipe is not None else None,
        "launches": agg["gemm"]["n"], "avg_ms": round(agg["gemm"]["ms"] / agg["gemm"]["n"], 4),
        "traffic": round(traffic) if traffic is not None else None,
        "traffic_note": ("DRAM read + write bytes per launch of the tracked ncu capture (profiles/), scaled by algorithmic bytes to the step's "
                         "average launch (%d MB algorithmic)" % round(alg / 1e6)) if traffic is not None else "no tracked ncu capture of the GEMM found",
    }
    if agg_sus is not None:
        gs = gemm_rate(agg_sus)
        roofline["sustained"] = {"achieved": round(gs, 1), "peak": round(sus_peak, 1), "frac": round(gs / sus_peak, 4),
                                 "frac_of_nominal_9pf": round(gs / NOMINAL_MXFP4_TFLOPS, 4),
                                 "peak_note": f"4 x {peaks['note']} bf16 cuBLAS SUSTAINED rate ({peaks['bf16_sustained']} TFLOP/s); per-launch events over >= {SUSTAINED_SECONDS:g} s of steps",
                                 "quantizers_GB/s": round(quant_rate(agg_sus)[0], 1)}
    sus_ms_step = sus_ms / sus_steps
    sustained = {"seconds": round(sus_ms / 1e3, 2), "steps": sus_steps, "ms_per_step": round(sus_ms_step, 4),
                 "value": round(flops / (sus_ms_step * 1e-3) / 1e12, 2), "clocks": sus_clocks,
                 "ms_x_mhz": round(sus_ms_step * sus_clocks["sm_mhz"], 1) if sus_clocks and sus_clocks.get("sm_mhz") else None,
                 "burst_ms_x_mhz": round(ms_per_step * clocks["sm_mhz"], 1) if clocks and clocks.get("sm_mhz") else None}
    h2d = sum(t.numel() * t.element_size() for t in xs_host + es_host)
    d2h = sum(t.numel() * t.element_size() for trio in out_host for t in trio)
    cpu_v, cpu_dt, cores, sample = cpu_arm(1, 0, layers_spec, tokens)
    out = {
        "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4",
        "data": "synthetic", "config": bench_config(args.workload, world, args.exchange),
        "e2e": {"value": round(flops / (e2e_ms / args.steps * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms / args.steps, 3),
                "GB/s_per_rank": {"h2d": round(h2d / (e2e_ms / args.steps * 1e-3) / 1e9, 1), "d2h": round(d2h / (e2e_ms / args.steps * 1e-3) / 1e9, 1)},
                "note": "per step: activations and grad-outputs copied from pinned host memory (side stream, one layer ahead of compute) and y, dx, "
                        "this rank's dW rows copied back into pinned host memory (second side stream); weights stay resident"},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": roofline,
        "roofline_quantizers": {"bound": "hbm", "achieved": round(q_gbs, 1), "peak": peaks["hbm"], "unit": "GB/s", "frac": round(q_gbs / peaks["hbm"], 4),
                                "peak_note": f"{peaks['note']} copy bandwidth",
                                "per_kernel": {k: {"GB/s": round(agg[k]["work"] / (agg[k]["ms"] * 1e-3) / 1e9, 1), "launches": agg[k]["n"],
                                                   "ms": round(agg[k]["ms"], 3)} for k in qn}},
        "time_share": {k: round(agg[k]["ms"] / sum(a["ms"] for a in agg.values()), 4) for k in agg},
        "sustained": sustained,
        "boundary_exceptions": exceptions,
        "cpu_baseline": {"value": round(cpu_v, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
                         "seconds": round(cpu_dt, 2)},
        "device_fault_word": status,
    }
    print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def model_step_arm(args):
    """One GPU, whole-model training step; prints tokens/s and the linear layers' share of it."""
    import torch

    import __graft_entry__ as entry

    entry.build()
    import quartet_b200.quantization as Q
    from quartet_b200 import ops
    from tests.llama_harness import TinyLlama

    torch.cuda.set_device(0)
    torch.manual_seed(0)
    batch, seq, vocab = 64, 512, 32000
    model = TinyLlama(Q, vocab=vocab, d=640, n_layer=6, n_head=5, multiple_of=256, eps=1e-5, fuse_producers=args.fuse_producers).cuda()
    step_model = torch.compile(model) if args.compile else model
    opt = torch.optim.AdamW(model.parameters(), lr=1.2e-3, fused=True)
    idx = torch.randint(0, vocab, (batch, seq), device="cuda")
    tgt = torch.randint(0, vocab, (batch, seq), device="cuda")

    def step():
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = step_model(idx, tgt)
            loss.backward()
        opt.step()
        return loss

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        loss = step()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.steps
    tokens = batch * seq
    lin_flops = sum(6.0 * tokens * k * n for k, n in ((640, 1920), (640, 640), (640, 3584), (1792, 640))) * 6
    print(json.dumps({
        "metric": "llama30m_train_step_tokens_per_s", "value": round(tokens / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 3), "higher_is_better": True, "dtype": "mxfp4 linears, bf16 autocast",
        "data": "synthetic", "compiled": bool(args.compile), "fuse_producers": bool(args.fuse_producers), "loss": round(loss.item(), 4),
        "config": {"workload": "llama30m_step", "model": "6 blocks, width 640, 5 heads, SwiGLU 1792, vocabulary 32000 (71 M parameters)",
                   "global_batch": batch, "seq_len": seq, "optimizer": "AdamW (fused)"},
        "quantized_linear_tflops_at_this_step_time": round(lin_flops / (ms * 1e-3) / 1e12, 1),
        "device_fault_word": ops.device_status(),
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=WORKLOAD, choices=sorted(WORKLOADS) + ["llama30m_step"])
    ap.add_argument("--compile", action="store_true", help="llama30m_step only: run the model under torch.compile")
    ap.add_argument("--fuse-producers", action="store_true",
                    help="llama30m_step only: RMSNorm and SwiGLU computed inside the forward quantizer of the layer they feed")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "copy", "nccl"],
                    help="wgrad exchange for --gpus > 1 (auto = copy: DMA engines push each owner's rows)")
    args = ap.parse_args()
    if args.workload == "llama30m_step":
        if args.impl == "reference" or int(os.environ.get("WORLD_SIZE", "1")) > 1:
            raise SystemExit("llama30m_step is a one-GPU workload of this library's arm")
        return model_step_arm(args)
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        w = WORKLOADS[args.workload]
        v, dt, cores, sample = cpu_arm(args.steps, args.warmup, w["layers"], w["tokens"])
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": round(v, 5), "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": bench_config(args.workload, args.gpus, args.exchange),
            "cpu_baseline": {"value": round(v, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(v, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }), flush=True)
        return
    args.warmup = max(args.warmup, 3)
    gpu_arm(args)


if __name__ == "__main__":
    main()
