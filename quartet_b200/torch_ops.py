"""The entry points as `torch.library` custom operators, `quartet_b200::*`, each with a fake (meta)
kernel that states its shape contract, so that the path can be traced and compiled
(`torch.compile(model)` is what the reference's production launch does: main_setup.sh:108 `--compile`,
src/optim/base.py:38-40).  The shape contracts are those the reference's notebook registers for the
real-quantized operators it calls (notebooks/benchmark_mxfp4.ipynb:881-958):

    quant_fwd       ~ fusedQuantizeMx        x[M,K]            -> e2m1[M,K/2], e8m0 blocked, mask[M,K/8]
    quant_bwd_t     ~ backward_t_bf16        g[M,N]            -> e2m1[N,M/2], e8m0 blocked
    requant_t       ~ backward_qt_bf16       e2m1[M,K/2], e8m0 -> e2m1[K,M/2], e8m0 blocked
    gemm_mxfp4_tn   ~ matmul_mxf4_bf16_tn    a[M,K/2], b[N,K/2], scales -> [M,N]

`linear_fwd` / `linear_bwd` are the whole QuantizedLinear forward / backward as ONE operator each
(what quantization/fused.py composes), registered with an autograd formula: a compiled model sees a
single opaque node per layer and direction, the Python random module and the quantizers' sign state
are touched only when the operator actually runs.

Every real kernel below is a call through the C ABI (quartet_b200.ops); there is no other
implementation behind these operators.
"""
from __future__ import annotations

import random
import weakref
from typing import Optional, Tuple

import torch

from . import ops

Tensor = torch.Tensor


def _sf_bytes(rows: int, cols: int) -> int:
    return ((rows + 127) // 128 * 128) * ((cols // 32 + 3) // 4 * 4)


def _u8(x: Tensor, *shape) -> Tensor:
    return x.new_empty(shape, dtype=torch.uint8)


# ------------------------------------------------------------------------------------------------
# quantizers
# ------------------------------------------------------------------------------------------------
@torch.library.custom_op("quartet_b200::quant_fwd", mutates_args=())
def quant_fwd(x: Tensor, had_scale: float, gaussian_scale: float) -> Tuple[Tensor, Tensor, Tensor]:
    codes, sf, mask = ops.quant_fwd(x, had_scale, gaussian_scale, return_mask=True)
    return codes, sf, mask


@quant_fwd.register_fake
def _(x, had_scale, gaussian_scale):
    rows, cols = x.shape
    return _u8(x, rows, cols // 2), _u8(x, _sf_bytes(rows, cols)), _u8(x, rows, cols // 8)


@torch.library.custom_op("quartet_b200::quant_bwd", mutates_args=())
def quant_bwd(x: Tensor, had_scale: float, signs: int, signs_dev: Optional[Tensor], rounding: int, seed: int, offset: int,
              noise: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    return ops.quant_bwd(x, had_scale, signs=signs, signs_dev=signs_dev, rounding=rounding, seed=seed, offset=offset, noise=noise)


@quant_bwd.register_fake
def _(x, had_scale, signs, signs_dev, rounding, seed, offset, noise):
    rows, cols = x.shape
    return _u8(x, rows, cols // 2), _u8(x, _sf_bytes(rows, cols))


@torch.library.custom_op("quartet_b200::quant_bwd_t", mutates_args=())
def quant_bwd_t(x: Tensor, had_scale: float, signs: int, signs_dev: Optional[Tensor], rounding: int, seed: int, offset: int,
                noise: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    return ops.quant_bwd_t(x, had_scale, signs=signs, signs_dev=signs_dev, rounding=rounding, seed=seed, offset=offset, noise=noise)


@quant_bwd_t.register_fake
def _(x, had_scale, signs, signs_dev, rounding, seed, offset, noise):
    rows, cols = x.shape
    return _u8(x, cols, rows // 2), _u8(x, _sf_bytes(cols, rows))


@torch.library.custom_op("quartet_b200::quant_bwd_dual", mutates_args=())
def quant_bwd_dual(x: Tensor, had_scale: float, signs: int, signs_dev: Optional[Tensor], rounding: int, seed_rows: int, seed_t: int,
                   offset: int) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    return ops.quant_bwd_dual(x, had_scale, signs=signs, signs_dev=signs_dev, rounding=rounding, seed_rows=seed_rows, seed_t=seed_t,
                              offset=offset)


@quant_bwd_dual.register_fake
def _(x, had_scale, signs, signs_dev, rounding, seed_rows, seed_t, offset):
    rows, cols = x.shape
    return (_u8(x, rows, cols // 2), _u8(x, _sf_bytes(rows, cols)), _u8(x, cols, rows // 2), _u8(x, _sf_bytes(cols, rows)))


@torch.library.custom_op("quartet_b200::requant_t", mutates_args=())
def requant_t(codes: Tensor, sf: Tensor, in_scale: float, had_scale: float, signs: int, signs_dev: Optional[Tensor], rounding: int,
              seed: int, offset: int, noise: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    return ops.requant_t(codes, sf, in_scale, had_scale, signs=signs, signs_dev=signs_dev, rounding=rounding, seed=seed, offset=offset,
                         noise=noise)


@requant_t.register_fake
def _(codes, sf, in_scale, had_scale, signs, signs_dev, rounding, seed, offset, noise):
    rows, cols = codes.shape[0], codes.shape[1] * 2
    return _u8(codes, cols, rows // 2), _u8(codes, _sf_bytes(cols, rows))


# ------------------------------------------------------------------------------------------------
# GEMM and the element-wise companions
# ------------------------------------------------------------------------------------------------
@torch.library.custom_op("quartet_b200::gemm_mxfp4_tn", mutates_args=())
def gemm_mxfp4_tn(a: Tensor, a_sf: Tensor, b: Tensor, b_sf: Tensor, alpha: float, mask: Optional[Tensor], had_scale: float,
                  out_dtype: torch.dtype) -> Tensor:
    return ops.gemm_mxfp4_tn(a, a_sf, b, b_sf, alpha, mask=mask, had_scale=had_scale, out_dtype=out_dtype)


@gemm_mxfp4_tn.register_fake
def _(a, a_sf, b, b_sf, alpha, mask, had_scale, out_dtype):
    torch._check(a.shape[1] == b.shape[1], lambda: "contraction extents differ")
    return a.new_empty((a.shape[0], b.shape[0]), dtype=out_dtype)


@torch.library.custom_op("quartet_b200::unrotate_mask", mutates_args=())
def unrotate_mask(g: Tensor, mask: Optional[Tensor], had_scale: float, out_dtype: torch.dtype) -> Tensor:
    return ops.unrotate_mask(g, mask, had_scale, out_dtype=out_dtype)


@unrotate_mask.register_fake
def _(g, mask, had_scale, out_dtype):
    return g.new_empty(g.shape, dtype=out_dtype)


@torch.library.custom_op("quartet_b200::dequant", mutates_args=())
def dequant(codes: Tensor, sf: Tensor, scale: float, out_dtype: torch.dtype) -> Tensor:
    return ops.dequant(codes, sf, scale, out_dtype)


@dequant.register_fake
def _(codes, sf, scale, out_dtype):
    return codes.new_empty((codes.shape[0], codes.shape[1] * 2), dtype=out_dtype)


# ------------------------------------------------------------------------------------------------
# the whole layer
# ------------------------------------------------------------------------------------------------
# A layer's quantizer modules carry state (the rotation's sign word, the rounding mode); operators take
# tensors and numbers only, so a layer is named by an integer handle.
_LAYERS: "weakref.WeakValueDictionary[int, torch.nn.Module]" = weakref.WeakValueDictionary()
_NEXT_HANDLE = [1]


def register_layer(layer: torch.nn.Module) -> int:
    handle = _NEXT_HANDLE[0]
    _NEXT_HANDLE[0] += 1
    _LAYERS[handle] = layer
    return handle


def _layer(handle: int):
    layer = _LAYERS.get(handle)
    if layer is None:
        raise RuntimeError(f"quartet_b200: no live QuantizedLinear with handle {handle}")
    return layer


def _pad128(n: int) -> int:
    return (n + 127) // 128 * 128


def _pad_rows(t: Tensor) -> Tensor:
    r = t.shape[0] % 128
    return t if r == 0 else torch.nn.functional.pad(t, (0, 0, 0, 128 - r))


@torch.library.custom_op("quartet_b200::linear_fwd", mutates_args=())
def linear_fwd(x: Tensor, w: Tensor, handle: int, out_dtype: torch.dtype) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """QuantizedLinear.forward of the production combination (src/models/quantization/__init__.py:36-42):
    y = Q_f(x) Q_f(w)^T on packed MXFP4 operands.  Returns y and what the backward needs: codes, scales and
    clip masks of both operands."""
    layer = _layer(handle)
    aq, wq = layer.activation_quantizer, layer.weight_quantizer
    aq._see(x)
    wq._see(w)
    K = w.shape[1]
    x2 = _pad_rows(x.reshape(-1, K).contiguous())
    if ops.FUSED_LAYER_CALLS:
        y, xc, xs, xm, wc, ws, wm = ops.linear_fwd(x2, w.contiguous(), aq.had_scale, wq.had_scale, out_dtype)
    else:
        xc, xs, xm = ops.quant_fwd(x2, aq.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=True)
        wc, ws, wm = ops.quant_fwd(w.contiguous(), wq.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=True)
        y = ops.gemm_mxfp4_tn(xc, xs, wc, ws, 1.0, out_dtype=out_dtype)
    m_real = x.numel() // K
    y = y[:m_real].reshape(*x.shape[:-1], w.shape[0])
    if m_real != y.shape[0] or not y.is_contiguous():
        y = y.contiguous()
    return y, xc, xs, xm, wc, ws, wm


@linear_fwd.register_fake
def _(x, w, handle, out_dtype):
    N, K = w.shape
    m = x.numel() // K
    mp = _pad128(m)
    return (x.new_empty((*x.shape[:-1], N), dtype=out_dtype), _u8(x, mp, K // 2), _u8(x, _sf_bytes(mp, K)), _u8(x, mp, K // 8),
            _u8(x, N, K // 2), _u8(x, _sf_bytes(N, K)), _u8(x, N, K // 8))


@torch.library.custom_op("quartet_b200::linear_bwd", mutates_args=())
def linear_bwd(e: Tensor, xc: Tensor, xs: Tensor, xm: Tensor, wc: Tensor, ws: Tensor, wm: Tensor, handle: int, x_dtype: torch.dtype,
               w_dtype: torch.dtype, need_dx: bool, need_dw: bool) -> Tuple[Tensor, Tensor]:
    """QEQWtt_QEtQXttFn.backward (src/models/quantization/backward.py:64-85) followed by the straight-through
    backward of both forward quantizers (mxfp4.py:142-146), on packed MXFP4 operands.  An output that is not
    needed comes back as an empty tensor."""
    layer = _layer(handle)
    aq, wq, g_q = layer.activation_quantizer, layer.weight_quantizer, layer.backward_scheme.g_quantizer
    N, K = wc.shape[0], wc.shape[1] * 2
    e2 = e.reshape(-1, N)
    m_real = e2.shape[0]
    if e2.dtype not in (torch.bfloat16, torch.float32):
        e2 = e2.float()
    e2 = _pad_rows(e2.contiguous())
    g_q._see(e2)
    g_q.re_randomize(device=e2.device)  # backward.py:69
    if g_q.stochastic:
        rounding = g_q.sr_rounding
        seeds = [random.randint(0, 1000000) for _ in range(4)]  # one per quantizer call, mxfp4_triton.py:196-197
    else:
        rounding, seeds = ops.ROUND_NEAREST, [0, 0, 0, 0]
    sg = g_q.sign_args()
    hb = g_q.had_scale
    alpha = (ops.SR_OPERAND_SCALE * g_q.out_scale) ** 2
    if ops.FUSED_LAYER_CALLS and rounding in (ops.ROUND_NEAREST, ops.ROUND_SR_PHILOX, ops.ROUND_SR_TLRAND):
        dx, dw = ops.linear_bwd(e2, xc, xs, xm, wc, ws, wm, hb, rounding, seeds, alpha, aq.had_scale, wq.had_scale, x_dtype, w_dtype, need_dx,
                                need_dw, **sg)
        if dx is not None and m_real != dx.shape[0]:
            dx = dx[:m_real].contiguous()
        if dx is None:
            dx = e.new_empty((0,), dtype=x_dtype)
        if dw is None:
            dw = e.new_empty((0,), dtype=w_dtype)
        ops.raise_on_fault("QuantizedLinear backward")  # only with QUARTET_CHECK_FAULTS=1
        return dx, dw
    dual = None
    if need_dx and need_dw and rounding in (ops.ROUND_NEAREST, ops.ROUND_SR_PHILOX):
        dual = ops.quant_bwd_dual(e2, hb, rounding=rounding, seed_rows=seeds[0], seed_t=seeds[2], **sg)
    dx = dw = None
    if need_dx:
        ec, es = dual[:2] if dual is not None else ops.quant_bwd(e2, hb, rounding=rounding, seed=seeds[0], **sg)
        wtc, wts = ops.requant_t(wc, ws, 1.0, hb, rounding=rounding, seed=seeds[1], **sg)
        dx = ops.gemm_mxfp4_tn(ec, es, wtc, wts, alpha, mask=xm, had_scale=aq.had_scale, out_dtype=x_dtype)
        if m_real != dx.shape[0]:
            dx = dx[:m_real].contiguous()
    if need_dw:
        etc, ets = dual[2:] if dual is not None else ops.quant_bwd_t(e2, hb, rounding=rounding, seed=seeds[2], **sg)
        xtc, xts = ops.requant_t(xc, xs, 1.0, hb, rounding=rounding, seed=seeds[3], **sg)
        dw = ops.gemm_mxfp4_tn(etc, ets, xtc, xts, alpha, mask=wm, had_scale=wq.had_scale, out_dtype=w_dtype)
    if dx is None:
        dx = e.new_empty((0,), dtype=x_dtype)
    if dw is None:
        dw = e.new_empty((0,), dtype=w_dtype)
    ops.raise_on_fault("QuantizedLinear backward")  # only with QUARTET_CHECK_FAULTS=1
    return dx, dw


@linear_bwd.register_fake
def _(e, xc, xs, xm, wc, ws, wm, handle, x_dtype, w_dtype, need_dx, need_dw):
    N, K = wc.shape[0], wc.shape[1] * 2
    m = e.numel() // N
    dx = e.new_empty((m, K), dtype=x_dtype) if need_dx else e.new_empty((0,), dtype=x_dtype)
    dw = e.new_empty((N, K), dtype=w_dtype) if need_dw else e.new_empty((0,), dtype=w_dtype)
    return dx, dw


def _linear_setup(ctx, inputs, output):
    x, w, handle, _ = inputs
    _, xc, xs, xm, wc, ws, wm = output
    ctx.save_for_backward(xc, xs, xm, wc, ws, wm)
    ctx.handle, ctx.x_shape, ctx.x_dtype, ctx.w_dtype = handle, x.shape, x.dtype, w.dtype
    ctx.set_materialize_grads(False)  # the six packed outputs never receive a gradient: no zero tensors for them


def _linear_backward(ctx, e, *unused):
    if e is None:
        return None, None, None, None
    xc, xs, xm, wc, ws, wm = ctx.saved_tensors
    need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    dx, dw = torch.ops.quartet_b200.linear_bwd(e.contiguous(), xc, xs, xm, wc, ws, wm, ctx.handle, ctx.x_dtype, ctx.w_dtype, need_dx, need_dw)
    return (dx.reshape(ctx.x_shape) if need_dx else None), (dw if need_dw else None), None, None


torch.library.register_autograd("quartet_b200::linear_fwd", _linear_backward, setup_context=_linear_setup)


def quantized_linear(x: Tensor, w: Tensor, handle: int, out_dtype: torch.dtype) -> Tensor:
    """y = QuantizedLinear(x) through the pair of operators above (differentiable, traceable)."""
    return torch.ops.quartet_b200.linear_fwd(x, w, handle, out_dtype)[0]
