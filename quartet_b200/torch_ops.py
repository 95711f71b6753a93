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


# ------------------------------------------------------------------------------------------------
# the layer with the forward quantizer fused into the elementwise step that produces its input
# ------------------------------------------------------------------------------------------------
def _weight_and_gemm(xc, xs, w, wq, out_dtype):
    wc, ws, wm = ops.quant_fwd(w.contiguous(), wq.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=True)
    return ops.gemm_mxfp4_tn(xc, xs, wc, ws, 1.0, out_dtype=out_dtype), wc, ws, wm


def _crop(y: Tensor, lead_shape, m_real: int, n: int) -> Tensor:
    y = y[:m_real].reshape(*lead_shape, n)
    return y if y.is_contiguous() else y.contiguous()


@torch.library.custom_op("quartet_b200::rmsnorm_linear_fwd", mutates_args=())
def rmsnorm_linear_fwd(x: Tensor, gamma: Tensor, eps: float, w: Tensor, handle: int,
                       out_dtype: torch.dtype) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """QuantizedLinear(RMSNorm(x)) with the norm of src/models/llama.py:64-75, `(x * rstd).type_as(x) * gamma`,
    computed inside the forward quantizer: the normalised activation (fp32, whatever the dtype of x) is never
    written.  Returns y, the packed operands the backward needs and rstd = rsqrt(mean(x^2) + eps) per row."""
    layer = _layer(handle)
    aq, wq = layer.activation_quantizer, layer.weight_quantizer
    aq._see(gamma)  # the quantizer's input is the fp32 product
    wq._see(w)
    K = w.shape[1]
    x2 = _pad_rows(x.reshape(-1, K).contiguous())
    xc, xs, xm, rstd = ops.quant_fwd_rmsnorm(x2, gamma.contiguous(), eps, aq.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=True)
    y, wc, ws, wm = _weight_and_gemm(xc, xs, w, wq, out_dtype)
    m_real = x.numel() // K
    return _crop(y, x.shape[:-1], m_real, w.shape[0]), xc, xs, xm, wc, ws, wm, rstd[:m_real].reshape(*x.shape[:-1], 1).contiguous()


@rmsnorm_linear_fwd.register_fake
def _(x, gamma, eps, w, handle, out_dtype):
    N, K = w.shape
    mp = _pad128(x.numel() // K)
    return (x.new_empty((*x.shape[:-1], N), dtype=out_dtype), _u8(x, mp, K // 2), _u8(x, _sf_bytes(mp, K)), _u8(x, mp, K // 8),
            _u8(x, N, K // 2), _u8(x, _sf_bytes(N, K)), _u8(x, N, K // 8), x.new_empty((*x.shape[:-1], 1), dtype=torch.float32))


def _rmsnorm_linear_setup(ctx, inputs, output):
    x, gamma, _, w, handle, _ = inputs
    _, xc, xs, xm, wc, ws, wm, rstd = output
    ctx.save_for_backward(xc, xs, xm, wc, ws, wm, rstd, x, gamma)
    ctx.handle, ctx.w_dtype = handle, w.dtype
    ctx.set_materialize_grads(False)


def _rmsnorm_linear_backward(ctx, e, *unused):
    if e is None:
        return None, None, None, None, None, None
    xc, xs, xm, wc, ws, wm, rstd, x, gamma = ctx.saved_tensors
    need_x, need_g, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[3]
    # gradient of the normalised activation (fp32), then the norm's own backward, step by step in the order autograd
    # differentiates `(xf * rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).type_as(x) * gamma`: the round-to-nearest
    # quantizers further up the backward pass turn a last-place difference in dx into different codes, so the
    # same operations in the same order are what keeps this path equal to the unfused model
    g, dw = torch.ops.quartet_b200.linear_bwd(e.contiguous(), xc, xs, xm, wc, ws, wm, ctx.handle, torch.float32, ctx.w_dtype,
                                              need_x or need_g, need_w)
    dx = dgamma = None
    if need_x or need_g:
        g = g.reshape(x.shape)
        xf = x.float()
        n_hat = (xf * rstd).type_as(x)
        if need_g:
            dgamma = (g * n_hat).sum(dim=tuple(range(g.dim() - 1))).to(gamma.dtype)
        if need_x:
            d_n = (g * gamma).to(x.dtype).float()                      # through `* gamma` and `.type_as(x)`
            d_r = (d_n * xf).sum(-1, keepdim=True)                      # n = xf * r
            d_m = (-0.5 * d_r) * rstd.pow(3)                            # r = rsqrt(m + eps)
            d_p = d_m.expand_as(xf) / xf.shape[-1]                      # m = mean(p)
            dx = (d_n * rstd + d_p * (2.0 * xf)).to(x.dtype)            # p = xf ** 2, both uses of xf
    return dx, dgamma, None, (dw if need_w else None), None, None


torch.library.register_autograd("quartet_b200::rmsnorm_linear_fwd", _rmsnorm_linear_backward, setup_context=_rmsnorm_linear_setup)


@torch.library.custom_op("quartet_b200::swiglu_linear_fwd", mutates_args=())
def swiglu_linear_fwd(h: Tensor, w: Tensor, handle: int, out_dtype: torch.dtype) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """QuantizedLinear(silu(up) * gate) with up, gate the two halves of h's last axis (src/models/llama.py:112-114),
    computed inside the forward quantizer: the product is never written."""
    layer = _layer(handle)
    aq, wq = layer.activation_quantizer, layer.weight_quantizer
    aq._see(h)
    wq._see(w)
    K = w.shape[1]
    h2 = _pad_rows(h.reshape(-1, 2 * K).contiguous())
    xc, xs, xm = ops.quant_fwd_swiglu(h2, aq.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=True)
    y, wc, ws, wm = _weight_and_gemm(xc, xs, w, wq, out_dtype)
    return _crop(y, h.shape[:-1], h.numel() // (2 * K), w.shape[0]), xc, xs, xm, wc, ws, wm


@swiglu_linear_fwd.register_fake
def _(h, w, handle, out_dtype):
    N, K = w.shape
    mp = _pad128(h.numel() // (2 * K))
    return (h.new_empty((*h.shape[:-1], N), dtype=out_dtype), _u8(h, mp, K // 2), _u8(h, _sf_bytes(mp, K)), _u8(h, mp, K // 8),
            _u8(h, N, K // 2), _u8(h, _sf_bytes(N, K)), _u8(h, N, K // 8))


def _swiglu_linear_setup(ctx, inputs, output):
    h, w, handle, _ = inputs
    _, xc, xs, xm, wc, ws, wm = output
    ctx.save_for_backward(xc, xs, xm, wc, ws, wm, h)
    ctx.handle, ctx.w_dtype = handle, w.dtype
    ctx.set_materialize_grads(False)


def _swiglu_linear_backward(ctx, e, *unused):
    if e is None:
        return None, None, None, None
    xc, xs, xm, wc, ws, wm, h = ctx.saved_tensors
    need_h, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    g, dw = torch.ops.quartet_b200.linear_bwd(e.contiguous(), xc, xs, xm, wc, ws, wm, ctx.handle, h.dtype, ctx.w_dtype, need_h, need_w)
    dh = None
    if need_h:
        # the operations autograd runs for `silu(up) * gate`, in h's dtype (see the note in the norm's backward)
        K = h.shape[-1] // 2
        g = g.reshape(*h.shape[:-1], K)
        up, gate = h[..., :K], h[..., K:]
        dh = torch.cat([torch.ops.aten.silu_backward(g * gate, up), g * torch.nn.functional.silu(up)], dim=-1)
    return dh, (dw if need_w else None), None, None


torch.library.register_autograd("quartet_b200::swiglu_linear_fwd", _swiglu_linear_backward, setup_context=_swiglu_linear_setup)
