"""Kernel-level micro-benchmark of the path, one kernel per run:

    python microbench.py --kernel quant_fwd  --rows 16384 --cols 4096 [--dtype bf16|f32]
    python microbench.py --kernel quant_fwd_rmsnorm --rows 16384 --cols 4096 --dtype f32   (rmsnorm_then_quant: the unfused sequence)
    python microbench.py --kernel quant_fwd_swiglu  --rows 16384 --cols 11008              (swiglu_then_quant: the unfused sequence)
    python microbench.py --kernel quant_bwd  --rows 16384 --cols 12288 [--rounding 1]
    python microbench.py --kernel quant_bwd_t --rows 16384 --cols 12288
    python microbench.py --kernel requant_t  --rows 16384 --cols 4096
    python microbench.py --kernel gemm --m 16384 --n 12288 --k 4096 [--fused-unrotate]
    python microbench.py --sweep            # quantize-only bandwidth sweep

Timing: CUDA events on the launching stream, `--warmup` untimed launches, then `--iters` timed
launches with a 256 MB write between launches to flush L2 (excluded from the timing).  Inputs are
Student-t(3) with 1 % of the channels scaled x20 (the quantize-sweep distribution) unless --gauss.
Prints one JSON line per case; quantizers report algorithmic GB/s, the GEMM TFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from quartet_b200 import ops  # noqa: E402

BYTES_PER_ELEM = {"quant_fwd": 0.5 + 1 / 32 + 1 / 8, "quant_fwd_rmsnorm": 0.5 + 1 / 32 + 1 / 8, "quant_fwd_swiglu": 0.5 + 1 / 32 + 1 / 8, "quant_bwd": 0.5 + 1 / 32, "quant_bwd_t": 0.5 + 1 / 32,
                  "quant_bwd_dual": 2 * (0.5 + 1 / 32)}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return json.load(open(path))
    except OSError:
        return {}


def make_input(rows, cols, dtype, gauss=False, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if gauss:
        return torch.randn(rows, cols, generator=g, device="cuda").to(dtype)
    # Student-t(3) = N / sqrt(chi2_3 / 3)
    z = torch.randn(rows, cols, generator=g, device="cuda")
    c = torch.randn(3, rows, cols, generator=g, device="cuda", dtype=torch.bfloat16).float().pow(2).sum(0) / 3
    x = z / c.sqrt()
    ch = torch.randperm(cols, generator=g, device="cuda")[: max(1, round(0.01 * cols))]
    x[:, ch] *= 20
    return x.to(dtype)


GRAPH_LAUNCHES = 0  # --graph N: time N back-to-back launches replayed from a CUDA graph (no host work between kernels)


def time_graph(fn, iters, warmup, n):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(n):
            fn()
    g.replay()
    torch.cuda.synchronize()
    best, total = float("inf"), 0.0
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        e.synchronize()
        ms = s.elapsed_time(e) / n
        total += ms
        best = min(best, ms)
    return total / iters, best


def time_kernel(fn, iters, warmup, flush=True):
    if GRAPH_LAUNCHES:
        return time_graph(fn, iters, warmup, GRAPH_LAUNCHES)
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    best = float("inf")
    for _ in range(iters):
        if flush:
            scratch.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        ms = s.elapsed_time(e)
        total += ms
        best = min(best, ms)
    return total / iters, best


def run_quant(kernel, rows, cols, dtype, rounding, iters, warmup, gauss, flush=True):
    esz = 2 if dtype == torch.bfloat16 else 4
    if kernel == "requant_t":
        x = make_input(rows, cols, torch.bfloat16, gauss)
        codes, sf, _ = ops.quant_fwd(x)
        del x
        fn = lambda: ops.requant_t(codes, sf, 1.0, rounding=rounding, seed=1)  # noqa: E731
        bytes_ = rows * cols * 2 * (0.5 + 1 / 32)
    else:
        x = make_input(rows, cols, dtype, gauss)
        if kernel == "quant_fwd":
            fn = lambda: ops.quant_fwd(x, ops.HAD_SCALE_BF16 if esz == 2 else ops.HAD_SCALE_F32)  # noqa: E731
        elif kernel in ("quant_fwd_rmsnorm", "rmsnorm_then_quant"):
            # cols = width of the normalised rows; bytes: the rows once (their second read is meant to come from L2)
            w = torch.ones(cols, device="cuda")
            if kernel == "quant_fwd_rmsnorm":
                fn = lambda: ops.quant_fwd_rmsnorm(x, w, 1e-5, ops.HAD_SCALE_F32)  # noqa: E731
            else:  # the unfused sequence, for comparison: torch's RMSNorm (llama.py:64-75 of the reference), then the plain quantizer
                fn = lambda: ops.quant_fwd((x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)).type_as(x) * w, ops.HAD_SCALE_F32)  # noqa: E731
            kernel_bytes = "quant_fwd_rmsnorm"
        elif kernel in ("quant_fwd_swiglu", "swiglu_then_quant"):
            # cols = hidden width; the input holds up and gate side by side
            del x
            x = make_input(rows, 2 * cols, dtype, True)
            if kernel == "quant_fwd_swiglu":
                fn = lambda: ops.quant_fwd_swiglu(x, ops.HAD_SCALE_BF16 if esz == 2 else ops.HAD_SCALE_F32)  # noqa: E731
            else:
                fn = lambda: ops.quant_fwd(torch.nn.functional.silu(x[:, :cols]) * x[:, cols:], ops.HAD_SCALE_BF16 if esz == 2 else ops.HAD_SCALE_F32)  # noqa: E731
            kernel_bytes = "quant_fwd_swiglu"
            esz *= 2
        elif kernel == "quant_bwd":
            fn = lambda: ops.quant_bwd(x, rounding=rounding, seed=1)  # noqa: E731
        elif kernel == "quant_bwd_dual":
            fn = lambda: ops.quant_bwd_dual(x, rounding=rounding, seed_rows=1, seed_t=2)  # noqa: E731
        else:
            fn = lambda: ops.quant_bwd_t(x, rounding=rounding, seed=1)  # noqa: E731
        bytes_ = rows * cols * (esz + BYTES_PER_ELEM[kernel_bytes if kernel not in BYTES_PER_ELEM else kernel])
    avg, best = time_kernel(fn, iters, warmup, flush)
    hbm = _peaks().get("hbm_gbs", 6650.0)
    gbs = bytes_ / (avg * 1e-3) / 1e9
    return {"kernel": kernel, "rows": rows, "cols": cols, "dtype": "bf16" if dtype == torch.bfloat16 else "f32", "rounding": rounding, "l2_flushed_between_launches": bool(flush),
            "avg_ms": round(avg, 4), "best_ms": round(best, 4), "GB/s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / hbm, 4),
            "algorithmic_bytes": int(bytes_)}


def run_gemm(m, n, k, iters, warmup, fused, out_f32, flush=True):
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randint(0, 256, (m, k // 2), generator=g, device="cuda", dtype=torch.uint8)
    b = torch.randint(0, 256, (n, k // 2), generator=g, device="cuda", dtype=torch.uint8)
    asf = torch.randint(118, 130, (ops.sf_bytes(m, k),), generator=g, device="cuda", dtype=torch.uint8)
    bsf = torch.randint(118, 130, (ops.sf_bytes(n, k),), generator=g, device="cuda", dtype=torch.uint8)
    mask = torch.randint(0, 256, (m, n // 8), generator=g, device="cuda", dtype=torch.uint8) if fused else None
    out = torch.empty(m, n, device="cuda", dtype=torch.float32 if out_f32 else torch.bfloat16)
    fn = lambda: ops.gemm_mxfp4_tn(a, asf, b, bsf, 16 / 9, mask=mask, out=out)  # noqa: E731
    avg, best = time_kernel(fn, iters, warmup, flush)
    p = _peaks()
    peak = 4 * p.get("bf16_tflops", 1590.0)
    tf = 2.0 * m * n * k / (avg * 1e-3) / 1e12
    return {"kernel": "gemm_mxfp4_tn", "m": m, "n": n, "k": k, "fused_unrotate": bool(fused), "out": "f32" if out_f32 else "bf16",
            "l2_flushed_between_launches": bool(flush), "avg_ms": round(avg, 4), "best_ms": round(best, 4), "TFLOP/s": round(tf, 1),
            "frac_of_4x_bf16_burst_peak": round(tf / peak, 4)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="quant_fwd", choices=["quant_fwd", "quant_fwd_rmsnorm", "rmsnorm_then_quant", "quant_fwd_swiglu", "swiglu_then_quant", "quant_bwd", "quant_bwd_t", "quant_bwd_dual", "requant_t", "gemm", "copy_ingress"])
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--rounding", type=int, default=ops.ROUND_SR_PHILOX)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--gauss", action="store_true")
    ap.add_argument("--fused-unrotate", action="store_true")
    ap.add_argument("--out-f32", action="store_true")
    ap.add_argument("--no-flush", action="store_true", help="do not flush L2 between launches (operands of the previous launch stay cached)")
    ap.add_argument("--graph", type=int, default=0, help="time N back-to-back launches replayed from a CUDA graph instead of single launches")
    ap.add_argument("--sweep", action="store_true", help="quantize-only sweep: K in {4096, 8192, 14336}, M = 4096 .. 131072")
    args = ap.parse_args()
    global GRAPH_LAUNCHES
    GRAPH_LAUNCHES = args.graph
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    if args.sweep:
        for k in (4096, 8192, 14336):
            m = 4096
            while m <= 131072:
                if m * k * 2 <= 6 << 30:
                    for kern in ("quant_fwd", "quant_bwd", "quant_bwd_t"):
                        print(json.dumps(run_quant(kern, m, k, torch.bfloat16, args.rounding, 5, 2, False)), flush=True)
                m *= 2
        return
    if args.kernel == "copy_ingress":
        # what one SM can take in through bulk copies: issuing threads x ring depth x copy size
        for producers, stages, chunk in ((1, 1, 16384), (1, 6, 16384), (2, 6, 16384), (4, 3, 16384), (2, 3, 32768), (4, 6, 8192)):
            v = ops.probe_copy_ingress(producers=producers, stages=stages, chunk=chunk)
            print(json.dumps({"kernel": "copy_ingress", "producers": producers, "stages": stages, "chunk": chunk,
                              "bytes_per_clk_per_sm": round(v, 1)}), flush=True)
        return
    if args.kernel == "gemm":
        print(json.dumps(run_gemm(args.m, args.n, args.k, args.iters, args.warmup, args.fused_unrotate, args.out_f32, not args.no_flush)))
    else:
        print(json.dumps(run_quant(args.kernel, args.rows, args.cols, dtype, args.rounding, args.iters, args.warmup, args.gauss, not args.no_flush)))


if __name__ == "__main__":
    main()
