"""Tensor-level wrappers over the C ABI.  torch supplies device memory and the
current stream; all arithmetic happens in libquartet_b200.so."""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib

BF16, F32 = 0, 1
ROUND_NEAREST, ROUND_SR_PHILOX, ROUND_SR_NOISE, ROUND_SR_TLRAND = 0, 1, 2, 3
QUEST_GAUSSIAN_SCALE = 2.92247856 / 6.0
HAD_SCALE_BF16 = 0.1767578125  # bf16(32 ** -0.5)
HAD_SCALE_F32 = 0.17677669529663687
SR_OPERAND_SCALE = 4.0 / 3.0  # each absmax-quantized operand carries this factor outside its scale bytes


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float32:
        return F32
    raise ValueError(f"dtype {t.dtype} not supported (bf16 or fp32)")


def _out_dt(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return BF16
    if dtype == torch.float32:
        return F32
    raise ValueError(f"output dtype {dtype} not supported (bf16 or fp32)")


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


_NO_SWITCH = _NoSwitch()


def _on(device):
    """Context that makes `device` current for the call; free when it already is (the one-process-per-GPU case)."""
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("tensors must live on a CUDA device")
        if t is not None and not t.is_contiguous():
            raise ValueError("tensors must be contiguous")


def sf_bytes(rows: int, cols: int) -> int:
    return ((rows + 127) // 128 * 128) * ((cols // 32 + 3) // 4 * 4)


def quant_fwd(x, had_scale=HAD_SCALE_BF16, gaussian_scale=QUEST_GAUSSIAN_SCALE, return_mask=True):
    """[rows, cols] -> (codes [rows, cols/2] u8, sf blocked u8, mask [rows, cols/8] u8 | None)."""
    _need_cuda(x)
    rows, cols = x.shape
    codes = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(rows, cols), dtype=torch.uint8, device=x.device)
    mask = torch.empty(rows, cols // 8, dtype=torch.uint8, device=x.device) if return_mask else None
    with _on(x.device):
        rc = _lib.load().quartet_quant_fwd(_ptr(x), _dt(x), rows, cols, had_scale, gaussian_scale, _ptr(codes), _ptr(sf),
                                           _ptr(mask), _stream())
    _lib.check(rc, "quartet_quant_fwd")
    return codes, sf, mask


def rms_stats(x, eps):
    """rsqrt(mean(x^2, -1) + eps) per row of [rows, cols] (bf16 / fp32) -> fp32 [rows]."""
    _need_cuda(x)
    rows, cols = x.shape
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    with _on(x.device):
        rc = _lib.load().quartet_rms_stats(_ptr(x), _dt(x), rows, cols, float(eps), _ptr(rstd), _stream())
    _lib.check(rc, "quartet_rms_stats")
    return rstd


def quant_fwd_rmsnorm(x, weight, eps, had_scale=HAD_SCALE_BF16, gaussian_scale=QUEST_GAUSSIAN_SCALE, return_mask=True):
    """Forward quantizer of RMSNorm(x) = (x * rstd).type_as(x) * weight without materialising it:
    [rows, cols], fp32 weight [cols] -> (codes, sf blocked, mask | None, rstd fp32 [rows])."""
    _need_cuda(x, weight)
    rows, cols = x.shape
    if weight.dtype != torch.float32 or weight.shape != (cols,) or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous fp32 vector with one entry per column")
    codes = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(rows, cols), dtype=torch.uint8, device=x.device)
    mask = torch.empty(rows, cols // 8, dtype=torch.uint8, device=x.device) if return_mask else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    with _on(x.device):
        rc = _lib.load().quartet_quant_fwd_rmsnorm(_ptr(x), _dt(x), rows, cols, _ptr(weight), float(eps), _ptr(rstd), had_scale, gaussian_scale,
                                                   _ptr(codes), _ptr(sf), _ptr(mask), _stream())
    _lib.check(rc, "quartet_quant_fwd_rmsnorm")
    return codes, sf, mask, rstd


def quant_fwd_swiglu(h, had_scale=HAD_SCALE_BF16, gaussian_scale=QUEST_GAUSSIAN_SCALE, return_mask=True):
    """Forward quantizer of silu(h[:, :H]) * h[:, H:] without materialising it: [rows, 2H] -> (codes [rows, H/2], sf, mask | None)."""
    _need_cuda(h)
    rows, two_h = h.shape
    if two_h % 2:
        raise ValueError("h must hold the up and gate halves side by side")
    hidden = two_h // 2
    codes = torch.empty(rows, hidden // 2, dtype=torch.uint8, device=h.device)
    sf = torch.empty(sf_bytes(rows, hidden), dtype=torch.uint8, device=h.device)
    mask = torch.empty(rows, hidden // 8, dtype=torch.uint8, device=h.device) if return_mask else None
    with _on(h.device):
        rc = _lib.load().quartet_quant_fwd_swiglu(_ptr(h), _dt(h), rows, hidden, had_scale, gaussian_scale, _ptr(codes), _ptr(sf), _ptr(mask),
                                                  _stream())
    _lib.check(rc, "quartet_quant_fwd_swiglu")
    return codes, sf, mask


def swiglu(h):
    """silu(h[:, :H]) * h[:, H:] written out, [rows, 2H] -> [rows, H] in h's dtype: the values quant_fwd_swiglu quantizes."""
    _need_cuda(h)
    rows, two_h = h.shape
    if two_h % 2:
        raise ValueError("h must hold the up and gate halves side by side")
    out = torch.empty(rows, two_h // 2, dtype=h.dtype, device=h.device)
    with _on(h.device):
        rc = _lib.load().quartet_swiglu(_ptr(h), _dt(h), rows, two_h // 2, _ptr(out), _stream())
    _lib.check(rc, "quartet_swiglu")
    return out


def _sr_args(signs, signs_dev, seed, offset, noise):
    return (int(signs) & 0xFFFFFFFF, _ptr(signs_dev)), (int(seed) & (2**64 - 1), int(offset) & (2**64 - 1), _ptr(noise))


def quant_bwd(x, had_scale=HAD_SCALE_BF16, signs=0, signs_dev=None, rounding=ROUND_SR_PHILOX, seed=0, offset=0, noise=None):
    """Row-wise backward quantizer: (codes [rows, cols/2], sf blocked); value = grid * 2^(sf-127) * 4/3."""
    _need_cuda(x, noise, signs_dev)
    rows, cols = x.shape
    codes = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(rows, cols), dtype=torch.uint8, device=x.device)
    (s, sd), (sd_, off, nz) = _sr_args(signs, signs_dev, seed, offset, noise)
    with _on(x.device):
        rc = _lib.load().quartet_quant_bwd(_ptr(x), _dt(x), rows, cols, had_scale, s, sd, rounding, sd_, off, nz, _ptr(codes),
                                           _ptr(sf), _stream())
    _lib.check(rc, "quartet_quant_bwd")
    return codes, sf


def quant_group32(x, kind, gaussian_scale=QUEST_GAUSSIAN_SCALE, rounding=ROUND_NEAREST, seed=0, offset=0, noise=None, return_mask=True):
    """Scaling + rounding + packing of an already rotated (or un-rotated) [rows, cols] tensor, groups of 32 along cols.
    kind 0: std-scaled round-to-nearest with clip mask -> (codes, sf, mask | None); kind 1: absmax-scaled -> (codes, sf, None)."""
    _need_cuda(x, noise)
    rows, cols = x.shape
    codes = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(rows, cols), dtype=torch.uint8, device=x.device)
    mask = torch.empty(rows, cols // 8, dtype=torch.uint8, device=x.device) if (kind == 0 and return_mask) else None
    m64 = 2**64 - 1
    with _on(x.device):
        rc = _lib.load().quartet_quant_group32(_ptr(x), _dt(x), rows, cols, kind, gaussian_scale, rounding, int(seed) & m64, int(offset) & m64,
                                               _ptr(noise), _ptr(codes), _ptr(sf), _ptr(mask), _stream())
    _lib.check(rc, "quartet_quant_group32")
    return codes, sf, mask


def quant_bwd_t(x, had_scale=HAD_SCALE_BF16, signs=0, signs_dev=None, rounding=ROUND_SR_PHILOX, seed=0, offset=0, noise=None):
    """Backward quantizer of x^T: (codes_t [cols, rows/2], sf_t blocked for [cols, rows/32])."""
    _need_cuda(x, noise, signs_dev)
    rows, cols = x.shape
    codes_t = torch.empty(cols, rows // 2, dtype=torch.uint8, device=x.device)
    sf_t = torch.empty(sf_bytes(cols, rows), dtype=torch.uint8, device=x.device)
    (s, sd), (sd_, off, nz) = _sr_args(signs, signs_dev, seed, offset, noise)
    with _on(x.device):
        rc = _lib.load().quartet_quant_bwd_t(_ptr(x), _dt(x), rows, cols, had_scale, s, sd, rounding, sd_, off, nz,
                                             _ptr(codes_t), _ptr(sf_t), _stream())
    _lib.check(rc, "quartet_quant_bwd_t")
    return codes_t, sf_t


def quant_bwd_dual(x, had_scale=HAD_SCALE_BF16, signs=0, signs_dev=None, rounding=ROUND_SR_PHILOX, seed_rows=0, seed_t=0, offset=0):
    """`quant_bwd(x, seed=seed_rows)` and `quant_bwd_t(x, seed=seed_t)` from one read of x:
    (codes, sf, codes_t, sf_t), bit-identical to the two separate calls."""
    _need_cuda(x, signs_dev)
    rows, cols = x.shape
    codes = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(rows, cols), dtype=torch.uint8, device=x.device)
    codes_t = torch.empty(cols, rows // 2, dtype=torch.uint8, device=x.device)
    sf_t = torch.empty(sf_bytes(cols, rows), dtype=torch.uint8, device=x.device)
    m64 = 2**64 - 1
    with _on(x.device):
        rc = _lib.load().quartet_quant_bwd_dual(_ptr(x), _dt(x), rows, cols, had_scale, int(signs) & 0xFFFFFFFF, _ptr(signs_dev), rounding,
                                                int(seed_rows) & m64, int(seed_t) & m64, int(offset) & m64, _ptr(codes), _ptr(sf),
                                                _ptr(codes_t), _ptr(sf_t), _stream())
    _lib.check(rc, "quartet_quant_bwd_dual")
    return codes, sf, codes_t, sf_t


def requant_t(codes, sf, in_scale=1.0, had_scale=HAD_SCALE_BF16, signs=0, signs_dev=None, rounding=ROUND_SR_PHILOX, seed=0,
              offset=0, noise=None):
    """MXFP4 [rows, cols] -> backward-quantized transpose (codes_t [cols, rows/2], sf_t)."""
    _need_cuda(codes, sf, noise, signs_dev)
    rows, cols = codes.shape[0], codes.shape[1] * 2
    codes_t = torch.empty(cols, rows // 2, dtype=torch.uint8, device=codes.device)
    sf_t = torch.empty(sf_bytes(cols, rows), dtype=torch.uint8, device=codes.device)
    (s, sd), (sd_, off, nz) = _sr_args(signs, signs_dev, seed, offset, noise)
    with _on(codes.device):
        rc = _lib.load().quartet_requant_t(_ptr(codes), _ptr(sf), rows, cols, in_scale, had_scale, s, sd, rounding, sd_, off,
                                           nz, _ptr(codes_t), _ptr(sf_t), _stream())
    _lib.check(rc, "quartet_requant_t")
    return codes_t, sf_t


def gemm_mxfp4_tn(a, a_sf, b, b_sf, alpha=1.0, mask=None, had_scale=HAD_SCALE_BF16, out_dtype=torch.bfloat16, out=None):
    """D[M,N] = alpha * A[M,K] . B[N,K]^T on packed e2m1 operands with blocked E8M0 scales."""
    _need_cuda(a, a_sf, b, b_sf, mask, out)
    M, K = a.shape[0], a.shape[1] * 2
    N = b.shape[0]
    if b.shape[1] * 2 != K:
        raise ValueError(f"contraction extents differ: {K} vs {b.shape[1] * 2}")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    with _on(a.device):
        rc = _lib.load().quartet_gemm_mxfp4_tn(_ptr(a), _ptr(a_sf), _ptr(b), _ptr(b_sf), M, N, K, alpha, _ptr(mask), had_scale,
                                               _ptr(out), _out_dt(out.dtype), _stream())
    _lib.check(rc, "quartet_gemm_mxfp4_tn")
    return out


# One host call per direction for the whole layer (quartet_linear_fwd / quartet_linear_bwd): the same kernels as the
# single entry points.  FUSED_LAYER_CALLS = False makes the layer code call the entry points one by one instead
# (what the benchmark's per-kernel timing pass does).
FUSED_LAYER_CALLS = True


def linear_fwd(x2, w, had_scale_x, had_scale_w, out_dtype, gaussian_scale=QUEST_GAUSSIAN_SCALE):
    """x2 [M, K] (M a multiple of 128), w [N, K] -> (y [M, N], xc, xs, xm, wc, ws, wm)."""
    _need_cuda(x2, w)
    M, K = x2.shape
    N = w.shape[0]
    dev = x2.device
    u8 = torch.uint8
    xc, xs, xm = torch.empty(M, K // 2, dtype=u8, device=dev), torch.empty(sf_bytes(M, K), dtype=u8, device=dev), torch.empty(M, K // 8, dtype=u8, device=dev)
    wc, ws, wm = torch.empty(N, K // 2, dtype=u8, device=dev), torch.empty(sf_bytes(N, K), dtype=u8, device=dev), torch.empty(N, K // 8, dtype=u8, device=dev)
    y = torch.empty(M, N, dtype=out_dtype, device=dev)
    with _on(dev):
        rc = _lib.load().quartet_linear_fwd(_ptr(x2), _dt(x2), _ptr(w), _dt(w), M, N, K, had_scale_x, had_scale_w, gaussian_scale, _ptr(xc), _ptr(xs),
                                            _ptr(xm), _ptr(wc), _ptr(ws), _ptr(wm), _ptr(y), _out_dt(out_dtype), _stream())
    _lib.check(rc, "quartet_linear_fwd")
    return y, xc, xs, xm, wc, ws, wm


def linear_bwd(e2, xc, xs, xm, wc, ws, wm, had_scale_b, rounding, seeds, alpha, had_scale_x, had_scale_w, x_dtype, w_dtype, need_dx=True,
               need_dw=True, signs=0, signs_dev=None, offset=0):
    """e2 [M, N] (M a multiple of 128) and the packed outputs of linear_fwd -> (dx [M, K] | None, dw [N, K] | None)."""
    _need_cuda(e2, xc, xs, xm, wc, ws, wm, signs_dev)
    M, N = e2.shape
    K = wc.shape[1] * 2
    dev = e2.device
    lib = _lib.load()
    work = torch.empty(lib.quartet_linear_bwd_workspace_bytes(M, N, K), dtype=torch.uint8, device=dev)
    dx = torch.empty(M, K, dtype=x_dtype, device=dev) if need_dx else None
    dw = torch.empty(N, K, dtype=w_dtype, device=dev) if need_dw else None
    m64 = 2**64 - 1
    seeds4 = (C.c_uint64 * 4)(*[int(v) & m64 for v in seeds])
    with _on(dev):
        rc = lib.quartet_linear_bwd(_ptr(e2), _dt(e2), M, N, K, _ptr(xc), _ptr(xs), _ptr(xm), _ptr(wc), _ptr(ws), _ptr(wm), had_scale_b,
                                    int(signs) & 0xFFFFFFFF, _ptr(signs_dev), rounding, seeds4, int(offset) & m64, alpha, had_scale_x, had_scale_w,
                                    _ptr(work), _ptr(dx), _out_dt(x_dtype), _ptr(dw), _out_dt(w_dtype), _stream())
    _lib.check(rc, "quartet_linear_bwd")
    return dx, dw


def gemm_mxfp4_tn_scatter(a, a_sf, b, b_sf, owner_ptrs, rows_per_owner, alpha=1.0, mask=None, had_scale=HAD_SCALE_BF16):
    """The fp32 product of `gemm_mxfp4_tn` with rows [o*rows_per_owner, (o+1)*rows_per_owner) stored to the
    device address owner_ptrs[o] (a dense [rows_per_owner, N] matrix, possibly in another GPU's memory)."""
    _need_cuda(a, a_sf, b, b_sf, mask)
    M, K = a.shape[0], a.shape[1] * 2
    N = b.shape[0]
    if b.shape[1] * 2 != K:
        raise ValueError(f"contraction extents differ: {K} vs {b.shape[1] * 2}")
    arr = (C.c_void_p * len(owner_ptrs))(*[int(x) for x in owner_ptrs])
    with _on(a.device):
        rc = _lib.load().quartet_gemm_mxfp4_tn_scatter(_ptr(a), _ptr(a_sf), _ptr(b), _ptr(b_sf), M, N, K, alpha, _ptr(mask), had_scale,
                                                       C.cast(arr, C.c_void_p), len(owner_ptrs), rows_per_owner, _stream())
    _lib.check(rc, "quartet_gemm_mxfp4_tn_scatter")


def shard_reduce(slots_ptr, n_slots, slot_elems, scale, out):
    """out[i] = scale * sum_s slots[s*slot_elems + i]; `slots_ptr` is a device address, `out` an fp32 tensor."""
    _need_cuda(out)
    if out.dtype != torch.float32 or not out.is_contiguous() or out.numel() != slot_elems:
        raise ValueError("out must be a contiguous fp32 tensor of slot_elems elements")
    with _on(out.device):
        rc = _lib.load().quartet_shard_reduce(int(slots_ptr), n_slots, slot_elems, scale, _ptr(out), _stream())
    _lib.check(rc, "quartet_shard_reduce")
    return out


def peer_alloc(nbytes, device):
    """(device address, 64-byte handle) of a buffer other processes of the node can map."""
    ptr, handle = C.c_void_p(), C.create_string_buffer(64)
    with torch.cuda.device(device):
        rc = _lib.load().quartet_peer_alloc(nbytes, C.byref(ptr), C.cast(handle, C.c_void_p))
    _lib.check(rc, "quartet_peer_alloc")
    return ptr.value, handle.raw


def peer_open(handle, device):
    ptr, buf = C.c_void_p(), C.create_string_buffer(bytes(handle), 64)
    with torch.cuda.device(device):
        rc = _lib.load().quartet_peer_open(C.cast(buf, C.c_void_p), C.byref(ptr))
    _lib.check(rc, "quartet_peer_open")
    return ptr.value


def peer_close(ptr, device):
    with torch.cuda.device(device):
        _lib.check(_lib.load().quartet_peer_close(int(ptr)), "quartet_peer_close")


def peer_copy(dst_ptr, src_ptr, nbytes, device):
    """Asynchronous copy between device addresses on the current stream (DMA engines, no SM)."""
    with torch.cuda.device(device):
        _lib.check(_lib.load().quartet_peer_copy(int(dst_ptr), int(src_ptr), nbytes, _stream()), "quartet_peer_copy")


def peer_free(ptr, device):
    with torch.cuda.device(device):
        _lib.check(_lib.load().quartet_peer_free(int(ptr)), "quartet_peer_free")


def probe_copy_ingress(region_mb=48, iters=4000, stages=6, chunk=16384, producers=2, device="cuda"):
    """Bytes per clock one SM takes in through bulk asynchronous copies (see csrc/probe_ingress.cu)."""
    src = torch.ones(region_mb << 20, dtype=torch.uint8, device=device)
    cycles = torch.zeros(1024, dtype=torch.int64, device=device)
    out = C.c_double(0.0)
    with torch.cuda.device(src.device):
        rc = _lib.load().quartet_probe_copy_ingress(_ptr(src), src.numel(), iters, stages, chunk, producers, _ptr(cycles), C.byref(out), _stream())
    _lib.check(rc, "quartet_probe_copy_ingress")
    return out.value


def probe_copy_ingress_noalloc(src, iters=4000, stages=6, chunk=16384, producers=2):
    """`probe_copy_ingress` on a caller-provided uint8 device tensor; neither this wrapper nor the library allocates."""
    _need_cuda(src)
    out = C.c_double(0.0)
    with torch.cuda.device(src.device):
        rc = _lib.load().quartet_probe_copy_ingress_noalloc(_ptr(src), src.numel() * src.element_size(), iters, stages, chunk, producers,
                                                            C.byref(out), _stream())
    _lib.check(rc, "quartet_probe_copy_ingress_noalloc")
    return out.value


def fold_signs(draw, word):
    """word (int64[1] or int32[1] device tensor, low 32 bits used) ^= bits j where draw[j] == 0; draw = the 32 zeros / ones
    of the reference's torch.randint(0, 2, (32,)) call (mxfp4.py:52-60), bf16 or fp32."""
    _need_cuda(draw, word)
    if draw.numel() != 32:
        raise ValueError("draw must hold 32 values")
    with _on(word.device):
        rc = _lib.load().quartet_fold_signs(_ptr(draw), _dt(draw), _ptr(word), _stream())
    _lib.check(rc, "quartet_fold_signs")
    return word


def unrotate_mask(g, mask=None, had_scale=HAD_SCALE_BF16, out_dtype=None):
    """((g * mask).view(-1, 32) @ H^T).view_as(g)"""
    _need_cuda(g, mask)
    out = torch.empty_like(g, dtype=out_dtype or g.dtype)
    cols = g.shape[-1]
    rows = g.numel() // cols
    with _on(g.device):
        rc = _lib.load().quartet_unrotate_mask(_ptr(g), _dt(g), _ptr(mask), rows, cols, had_scale, _ptr(out), _out_dt(out.dtype),
                                               _stream())
    _lib.check(rc, "quartet_unrotate_mask")
    return out


def dequant(codes, sf, scale=1.0, dtype=torch.float32):
    """codes [rows, cols/2] + blocked sf -> [rows, cols] values grid * 2^(sf-127) * scale."""
    _need_cuda(codes, sf)
    rows, cols = codes.shape[0], codes.shape[1] * 2
    out = torch.empty(rows, cols, dtype=dtype, device=codes.device)
    with _on(codes.device):
        rc = _lib.load().quartet_dequant(_ptr(codes), _ptr(sf), rows, cols, scale, _ptr(out), _out_dt(dtype), _stream())
    _lib.check(rc, "quartet_dequant")
    return out


def device_status() -> int:
    """Fault word of the current device (0 = no kernel ever gave up on a bounded wait); clears it."""
    st = C.c_int32(0)
    _lib.check(_lib.load().quartet_device_status(C.byref(st)), "quartet_device_status")
    return st.value


# Every wait inside the kernels is bounded: a kernel that gives up leaves its tiles unwritten and records the
# fact in the fault word instead of hanging.  Nothing reads that word on the hot path (it costs a device
# synchronisation), so a caller that wants wrong results turned into an exception either polls device_status()
# itself at a point where it synchronises anyway, or sets QUARTET_CHECK_FAULTS=1: the layer's backward and
# the gradient exchange's wait() then check the word and raise.
CHECK_FAULTS = os.environ.get("QUARTET_CHECK_FAULTS", "0") not in ("", "0")


def raise_on_fault(where: str) -> None:
    if CHECK_FAULTS:
        word = device_status()
        if word:
            raise _lib.QuartetError(f"{where}: a kernel gave up on a bounded wait (fault word {word:#x}); its results are incomplete")


def unpack_mask(mask_u8: torch.Tensor) -> torch.Tensor:
    """[rows, cols/8] bit-packed (LSB first) -> bool [rows, cols]  (benchmark_mxfp4.ipynb:975-979 `_unpack_mask`)."""
    bits = torch.arange(8, device=mask_u8.device, dtype=torch.uint8)
    return ((mask_u8.unsqueeze(-1) >> bits) & 1).bool().reshape(*mask_u8.shape[:-1], mask_u8.shape[-1] * 8)
