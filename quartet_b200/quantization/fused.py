"""The production combination as ONE autograd function on real MXFP4 data:

    weight/activation quantizer  QuestMXFP4Quantizer
    gradient quantizer           AlbertTsengQuantizer / AlignedAlbertTsengQuantizer
    backward scheme              "Q(E)Q(Wt)t_Q(Et)Q(Xt)t"

It computes what QuantizedLinear.forward (src/models/quantization/__init__.py:36-42) followed by
QEQWtt_QEtQXttFn.backward (backward.py:64-85) and the two QuestMXFP4QuantizerFn.backward calls
(mxfp4.py:142-146) compute, but keeps operands as packed e2m1 + E8M0 from quantizer to GEMM:

    forward   Xq = Q_f(X), Wq = Q_f(W)                    -> Y  = Xq Wq^T
    backward  Q_b(E), Q_b(Wq^T)   (contraction over N)    -> dX = unrotate(mask_x * 16/9 * ...)
              Q_b(E^T), Q_b(Xq^T) (contraction over M)    -> dW = unrotate(mask_w * 16/9 * ...)

Saved for backward: codes, scales and bit masks only (4.4 bits per element instead of 16/32).
"""
from __future__ import annotations

import random

import torch

from .. import ops


def _pad_rows(t: torch.Tensor, mult: int = 128) -> torch.Tensor:
    r = t.shape[0] % mult
    if r == 0:
        return t
    return torch.nn.functional.pad(t, (0, 0, 0, mult - r))


class QuartetLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, a_q, w_q, g_q, out_dtype, wgrad_sink=None):
        K = w.shape[1]
        x2 = x.reshape(-1, K)
        m_real = x2.shape[0]
        x2 = _pad_rows(x2.contiguous())
        wc_ = w.contiguous()
        if ops.FUSED_LAYER_CALLS:  # one host call for the three launches
            y, xc, xs, xm, wc, ws, wm = ops.linear_fwd(x2, wc_, a_q.had_scale, w_q.had_scale, out_dtype)
        else:
            xc, xs, xm = ops.quant_fwd(x2, a_q.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=True)
            wc, ws, wm = ops.quant_fwd(wc_, w_q.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=True)
            y = ops.gemm_mxfp4_tn(xc, xs, wc, ws, 1.0, out_dtype=out_dtype)
        ctx.save_for_backward(xc, xs, xm, wc, ws, wm)
        ctx.a_q, ctx.w_q, ctx.g_q = a_q, w_q, g_q
        ctx.x_shape, ctx.m_real = x.shape, m_real
        ctx.x_dtype, ctx.w_dtype = x.dtype, w.dtype
        ctx.wgrad_sink, ctx.weight = wgrad_sink, w
        return y[:m_real].reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, e):
        xc, xs, xm, wc, ws, wm = ctx.saved_tensors
        g_q = ctx.g_q
        N = wc.shape[0]
        e2 = e.reshape(-1, N)
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
        if ops.FUSED_LAYER_CALLS and ctx.wgrad_sink is None and rounding in (ops.ROUND_NEAREST, ops.ROUND_SR_PHILOX, ops.ROUND_SR_TLRAND):
            dx, dw = ops.linear_bwd(e2, xc, xs, xm, wc, ws, wm, hb, rounding, seeds, alpha, ctx.a_q.had_scale, ctx.w_q.had_scale, ctx.x_dtype,
                                    ctx.w_dtype, ctx.needs_input_grad[0], ctx.needs_input_grad[1], **sg)
            if dx is not None:
                dx = dx[:ctx.m_real].reshape(ctx.x_shape)
            return dx, dw, None, None, None, None, None
        dx = dw = None
        dual = None
        if ctx.needs_input_grad[0] and ctx.needs_input_grad[1] and rounding in (ops.ROUND_NEAREST, ops.ROUND_SR_PHILOX):
            # one read of E for both of its quantizations (same bits as the two separate calls below)
            dual = ops.quant_bwd_dual(e2, hb, rounding=rounding, seed_rows=seeds[0], seed_t=seeds[2], **sg)
        if ctx.needs_input_grad[0]:
            ec, es = dual[:2] if dual is not None else ops.quant_bwd(e2, hb, rounding=rounding, seed=seeds[0], **sg)
            wtc, wts = ops.requant_t(wc, ws, 1.0, hb, rounding=rounding, seed=seeds[1], **sg)
            dx = ops.gemm_mxfp4_tn(ec, es, wtc, wts, alpha, mask=xm, had_scale=ctx.a_q.had_scale, out_dtype=ctx.x_dtype)
            dx = dx[:ctx.m_real].reshape(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            etc, ets = dual[2:] if dual is not None else ops.quant_bwd_t(e2, hb, rounding=rounding, seed=seeds[2], **sg)
            xtc, xts = ops.requant_t(xc, xs, 1.0, hb, rounding=rounding, seed=seeds[3], **sg)
            sink = ctx.wgrad_sink
            if sink is not None and sink.accepts(wc.shape[0], wc.shape[1] * 2, ctx.w_dtype):
                # the GEMM delivers each rank's rows to their owner; the averaged shard lands in weight.grad_shard
                sink.wgrad(ctx.weight, etc, ets, xtc, xts, alpha, wm, ctx.w_q.had_scale)
            else:
                dw = ops.gemm_mxfp4_tn(etc, ets, xtc, xts, alpha, mask=wm, had_scale=ctx.w_q.had_scale, out_dtype=ctx.w_dtype)
        return dx, dw, None, None, None, None, None
