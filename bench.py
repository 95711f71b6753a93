"""Benchmark of the MXFP4 quantized-linear path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("llama7b_linears_16384tok"): the four linear layers of a 7B Llama block
(QKV 4096->12288, O 4096->4096, gate/up 4096->22016, down 11008->4096), forward + dgrad + wgrad,
16384 tokens per GPU, bf16 activations ~N(0,1), fp32 master weights ~N(0,0.02), bf16 grad-outputs
~N(0,1e-3); synthetic, seeded.  One step = all four layers once, through
quartet_b200.quantization.QuantizedLinear (forward + backward).  Token rows are sharded over the
GPUs (weak scaling: 16384 tokens on every GPU); the per-GPU weight-gradient partials are averaged
inside the step, every rank ending up with its row shard (--exchange: rows pushed into their owner's
memory by the DMA engines or by the GEMM's own stores, or an NCCL reduce-scatter).  Metric: model FLOP/s = 6*M*N*K per layer, summed over
layers and GPUs.

`--impl reference` times the reference's own pseudo-quantized arithmetic for the same layers on the
host CPU (the torch-fp32 restatement in oracle/ref_math.py, which is pinned bit-exactly to the
reference kernel) on a bounded token sample.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = [("qkv", 4096, 12288), ("o", 4096, 4096), ("gate_up", 4096, 22016), ("down", 11008, 4096)]
TOKENS = 16384
CPU_SAMPLE_TOKENS = int(os.environ.get("QUARTET_BENCH_CPU_TOKENS", "512"))  # token sample of the CPU arm (the tests shrink it)
WORKLOAD = "llama7b_linears_16384tok"
METRIC = "quantized_linear_fwd_bwd_tflops"


# DRAM traffic of the GEMM, from the ncu capture summarised in profiles/gemm_mxfp4_2cta_8192x8192x4096.md
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch).  The bench's launches are larger than the
# capture rule allows, so the captured traffic is scaled by algorithmic bytes (operands + scales + result).
NCU_GEMM_CAPTURE = {"m": 8192, "n": 8192, "k": 4096, "out_bytes": 2, "dram_bytes": 36.13e6 + 84.27e6}


def gemm_algorithmic_bytes(m, n, k, out_bytes):
    return (m + n) * k * (0.5 + 1.0 / 32.0) + m * n * out_bytes


def gemm_traffic_per_launch(tokens):
    """Average over the 12 GEMM launches of a step (forward and dgrad write bf16, wgrad fp32)."""
    cap = NCU_GEMM_CAPTURE
    ratio = cap["dram_bytes"] / gemm_algorithmic_bytes(cap["m"], cap["n"], cap["k"], cap["out_bytes"])
    alg = 0.0
    for _, k, n in LAYERS:
        alg += gemm_algorithmic_bytes(tokens, n, k, 2) + gemm_algorithmic_bytes(tokens, k, n, 2) + gemm_algorithmic_bytes(n, k, tokens, 4)
    return ratio * alg / (3 * len(LAYERS)), alg / (3 * len(LAYERS))


def layer_flops(m):
    return sum(6.0 * m * k * n for _, k, n in LAYERS)


# ----------------------------------------------------------------------------------------------
# CPU arm (the reference's arithmetic on host cores)
# ----------------------------------------------------------------------------------------------
def cpu_arm(steps, warmup, tokens=CPU_SAMPLE_TOKENS):
    import torch

    from oracle import ref_math as rm

    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(0)
    data = []
    for _, k, n in LAYERS:
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
    return layer_flops(tokens) / dt / 1e12, dt, cores, f"{tokens} of {TOKENS} tokens per layer, all four layers, fp32 torch ops"


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
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

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
# GPU arm
# ----------------------------------------------------------------------------------------------
def gpu_arm(args):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

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
    from quartet_b200.staging import HostStager

    # ---- model + data (seeded; weights identical on every rank, activations differ per rank) ----
    gw = torch.Generator(device="cpu").manual_seed(0)
    layers, xs, es, xs_host, es_host = [], [], [], [], []
    for _, k, n in LAYERS:
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
    for _, k, n in LAYERS:
        xh = torch.randn(TOKENS, k, dtype=torch.bfloat16).pin_memory()
        eh = (torch.randn(TOKENS, n) * 1e-3).to(torch.bfloat16).pin_memory()
        xs_host.append(xh), es_host.append(eh)
        xs.append(xh.to(dev).requires_grad_(True)), es.append(eh.to(dev))
    # wgrad exchange across ranks: rows of each partial dW go straight from the GEMM epilogue into their
    # owner's memory ("peer", the default), or a NCCL reduce-scatter of full partials ("nccl")
    reducer = sink = None
    if args.exchange == "auto":
        # measured on 2 and on 8 GPUs: the DMA-engine push costs less than the slowdown of a GEMM whose epilogue
        # stores cross NVLink
        args.exchange = "copy"
    if world > 1 and args.exchange in ("peer", "copy"):
        try:
            sink = PeerWgradScatter(device=dev, transport="store" if args.exchange == "peer" else "copy")
            for lin in layers:
                sink.prepare(lin.weight)
            for lin in layers:
                lin.wgrad_sink = sink
        except PeerSetupError as exc:  # raised on every rank alike: fall back to the library collective everywhere
            if rank == 0:
                print(f"bench: {exc}; using the NCCL reduce-scatter", file=sys.stderr)
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

    real = {n: getattr(ops, n) for n in ("quant_fwd", "quant_bwd", "quant_bwd_t", "requant_t", "gemm_mxfp4_tn")}
    ops.quant_fwd = wrap("quant_fwd", real["quant_fwd"], q_bytes(0.53125, 0.125))
    ops.quant_bwd = wrap("quant_bwd", real["quant_bwd"], lambda x, *a, **k: ("bytes", x.numel() * (x.element_size() + 0.53125)))
    ops.quant_bwd_t = wrap("quant_bwd_t", real["quant_bwd_t"], lambda x, *a, **k: ("bytes", x.numel() * (x.element_size() + 0.53125)))
    ops.quant_bwd_dual = wrap("quant_bwd_dual", ops.quant_bwd_dual, lambda x, *a, **k: ("bytes", x.numel() * (x.element_size() + 2 * 0.53125)))
    ops.requant_t = wrap("requant_t", real["requant_t"], lambda c, *a, **k: ("bytes", c.numel() * 2 * 1.0625))
    ops.gemm_mxfp4_tn_scatter = wrap("gemm", ops.gemm_mxfp4_tn_scatter,
                                     lambda a_, asf, b_, *r, **k: ("flops", 2.0 * a_.shape[0] * b_.shape[0] * a_.shape[1] * 2))
    ops.shard_reduce = wrap("shard_reduce", ops.shard_reduce, lambda ptr, n_slots, elems, *r, **k: ("bytes", (n_slots + 1) * elems * 4))
    ops.gemm_mxfp4_tn = wrap("gemm", real["gemm_mxfp4_tn"],
                             lambda a_, asf, b_, *r, **k: ("flops", 2.0 * a_.shape[0] * b_.shape[0] * a_.shape[1] * 2))

    stager = HostStager(dev)
    for i in range(len(LAYERS)):
        stager.register(i, (xs[i], es[i]))
    pending = {"items": 0}  # how many (step, layer) items of the current timed run are still to be prefetched

    def prefetch_next(i):
        if pending["items"] > 0:
            pending["items"] -= 1
            stager.prefetch(i, (xs_host[i], es_host[i]))

    def step(from_host=False):
        sums = []
        for i, lin in enumerate(layers):
            if from_host:
                stager.acquire(i)                       # compute stream waits for this layer's inputs
                prefetch_next((i + 1) % len(layers))    # next layer's (or next step's first) inputs cross PCIe meanwhile
            xs[i].grad = None
            lin.weight.grad = None
            y = lin(xs[i])
            y.backward(es[i])
            if reducer is not None:
                reducer.submit(lin.weight.grad)
            if from_host:
                sums.append([y.float().sum(), xs[i].grad.float().sum()])
                stager.release(i)
        shards = reducer.wait() if reducer is not None else (sink.wait() if sink is not None else [lin.weight.grad for lin in layers])
        if from_host:
            # the step's result read back to the host: per-layer checksums of y, dx and this rank's dw (shard)
            return torch.stack([torch.stack(s2 + [dw.float().sum()]) for s2, dw in zip(sums, shards)]).cpu()
        return None

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
        e.record()
        torch.cuda.synchronize()
        ms = torch.tensor([s.elapsed_time(e)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.barrier()
        return ms.item()

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(torch.cuda.current_device() if os.environ.get("CUDA_VISIBLE_DEVICES") is None else int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    if rank == 0:
        sampler.start()
    counts["n"] = 0
    total_ms = timed(args.steps, False)
    launches = counts["n"]
    clocks = sampler.stop() if rank == 0 else None

    timed(1, True)
    e2e_ms = timed(args.steps, True)

    # ---- per-kernel timing (live, CUDA events on the launching stream, outside the headline region) ----
    timing["on"] = True
    for _ in range(max(2, min(args.steps, 5))):
        step()
    torch.cuda.synchronize()
    timing["on"] = False
    agg = {}
    for name, s, e, (kind, work) in timing["rec"]:
        a = agg.setdefault(name, {"ms": 0.0, "work": 0.0, "kind": kind, "n": 0})
        a["ms"] += s.elapsed_time(e)
        a["work"] += work
        a["n"] += 1
    status = ops.device_status()
    if sink is not None:
        sink.close()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    bf16_peak = peaks.get("bf16_tflops_sustained", 1400.0)
    peak_note = "measured" if peaks else "fallback"
    ms_per_step = total_ms / args.steps
    flops = layer_flops(TOKENS) * world
    value = flops / (ms_per_step * 1e-3) / 1e12
    g = agg["gemm"]
    gemm_tflops = g["work"] / (g["ms"] * 1e-3) / 1e12
    qn = [k for k in agg if k != "gemm"]
    q_ms = sum(agg[k]["ms"] for k in qn)
    q_gbs = sum(agg[k]["work"] for k in qn) / (q_ms * 1e-3) / 1e9
    h2d = sum(t.numel() * t.element_size() for t in xs_host + es_host)
    cpu_v, cpu_dt, cores, sample = cpu_arm(1, 0)
    out = {
        "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_gpu": TOKENS, "layers": [[n_, k, n] for n_, k, n in LAYERS],
                   "activations": "bf16", "weights": "fp32 master", "parallelism": f"dp{world} token-row shards" + ("" if world == 1 else {"peer": " + wgrad rows stored to their owner by the GEMM (peer memory)", "copy": " + wgrad rows pushed to their owner by the DMA engines", "nccl": " + NCCL reduce-scatter of wgrad"}[args.exchange]),
                   "l2": "inputs larger than L2 (>= 134 MB per operand, 3.9 GB per step)"},
        "e2e": {"value": round(flops / (e2e_ms / args.steps * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": len(LAYERS) * 3 * 4, "ms_per_step": round(e2e_ms / args.steps, 3),
                "note": "activations and grad-outputs copied from pinned host memory every step (side stream, one layer ahead of compute); weights stay resident; per-layer checksums of y, dx, dw read back"},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "gemm_mxfp4_2cta_kernel", "achieved": round(gemm_tflops, 1), "peak": round(4 * bf16_peak, 1),
                     "unit": "TFLOP/s", "frac": round(gemm_tflops / (4 * bf16_peak), 4), "traffic": round(gemm_traffic_per_launch(TOKENS)[0]),
                     "traffic_note": "DRAM bytes per launch: ncu capture of 8192x8192x4096 (120.4 MB) scaled by algorithmic bytes to the step's average launch (%d MB algorithmic)" % round(gemm_traffic_per_launch(TOKENS)[1] / 1e6),
                     "peak_note": f"4 x {peak_note} sustained bf16 cuBLAS rate (MXFP4:bf16 dense ratio of the tensor cores)",
                     "launches": g["n"], "avg_ms": round(g["ms"] / g["n"], 4)},
        "roofline_quantizers": {"bound": "hbm", "achieved": round(q_gbs, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(q_gbs / hbm_peak, 4),
                                "peak_note": f"{peak_note} copy bandwidth",
                                "per_kernel": {k: {"GB/s": round(agg[k]["work"] / (agg[k]["ms"] * 1e-3) / 1e9, 1), "launches": agg[k]["n"],
                                                   "ms": round(agg[k]["ms"], 3)} for k in qn}},
        "time_share": {k: round(agg[k]["ms"] / sum(a["ms"] for a in agg.values()), 4) for k in agg},
        "cpu_baseline": {"value": round(cpu_v, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
                         "seconds": round(cpu_dt, 2)},
        "device_fault_word": status,
    }
    print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "copy", "nccl"],
                    help="wgrad exchange for --gpus > 1 (auto = copy: DMA engines push each owner's rows)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        steps = min(args.steps, 5)
        v, dt, cores, sample = cpu_arm(steps, min(args.warmup, 1))
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": round(v, 5), "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": min(args.warmup, 1), "ms_per_step": round(dt * 1e3, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu": TOKENS, "layers": [[n_, k, n] for n_, k, n in LAYERS]},
            "cpu_baseline": {"value": round(v, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(v, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }), flush=True)
        return
    gpu_arm(args)


if __name__ == "__main__":
    main()
