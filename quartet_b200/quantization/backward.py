"""Backward schemes under the reference's names (src/models/quantization/backward.py:97-101):

    "EW_EtX"                    plain gradients, nothing quantized in the backward pass
    "Q(E)W_Q(Et)X"              the output-gradient is quantized for both products, W and X are not
    "Q(E)Q(Wt)t_Q(Et)Q(Xt)t"    all four operands of the two backward GEMMs are quantized

A scheme is a module with a `g_quantizer` attribute (assigned by QuantizedLinear) and `forward(x, w)`.
When `g_quantizer` is one of this library's absmax quantizers and the shapes allow it, the backward
quantizations run as the library's kernels on PACKED operands (no transposed copy is materialised:
`quant_bwd_t` quantizes E^T, W^T, X^T straight from E, W, X) and the fully quantized scheme multiplies
them with the block-scaled MXFP4 GEMM.  The half-quantized scheme has one MXFP4 operand and one dense
operand per product; a mixed MXFP4 x bf16 GEMM is not built, so its quantized operand is de-quantized
(`dequant`) and the product is an ordinary matmul.  Any other gradient quantizer (NoQuantizer, a class of
the reference) is applied as a module, on materialised transposes, as the reference applies it.

QuantizedLinear short-cuts the production combination (forward quantizers included) into fused.py /
torch_ops.py; the functions here serve every other combination.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.autograd import Function

from .. import ops


def _packable(g, *mats) -> bool:
    """True when `g` can emit packed MXFP4 for these 2-D operands through the library's kernels."""
    from .quantizers import AbsmaxRotation32

    return (isinstance(g, AbsmaxRotation32)
            and all(m.is_cuda and m.dtype in (torch.bfloat16, torch.float32) and m.shape[0] % 128 == 0 and m.shape[1] % 128 == 0 for m in mats))


def _flat2d(t: torch.Tensor) -> torch.Tensor:
    return t.reshape(-1, t.shape[-1]).contiguous()


class EW_EtX_Scheme(nn.Module):
    """No quantization in the backward pass: autograd's own dX = E W, dW = E^T X."""

    def __init__(self):
        super().__init__()
        self.g_quantizer = None

    def forward(self, x, w):
        return torch.nn.functional.linear(x, w)


class QEW_QEtXFn(Function):
    """dX = Q(E) W and dW = Q(E^T) X: only the output-gradient is quantized."""

    @staticmethod
    def forward(ctx, x, w, g_quantizer):
        ctx.save_for_backward(x, w)
        ctx.g = g_quantizer
        return torch.nn.functional.linear(x, w)

    @staticmethod
    def backward(ctx, e):
        x, w = ctx.saved_tensors
        g = ctx.g
        e2, x2 = _flat2d(e), _flat2d(x)
        if _packable(g, e2):
            # Q(E) and Q(E^T) come out of the kernels as MXFP4; the other operand of each product is dense, so the
            # quantized one is expanded again and the product is a dense matmul
            g._see(e2)
            scale = ops.SR_OPERAND_SCALE * g.out_scale
            qe = ops.dequant(*g.pack(e2), scale, e2.dtype)
            qet = ops.dequant(*g.pack_t(e2), scale, e2.dtype)
        else:
            qe, qet = g(e2), g(e2.t().contiguous())
        dx = (qe @ w.to(qe.dtype)).reshape(x.shape)
        dw = qet @ x2.to(qet.dtype)
        return dx, dw, None


class QEW_QEtX_Scheme(EW_EtX_Scheme):
    def forward(self, x, w):
        return QEW_QEtXFn.apply(x, w, self.g_quantizer)


class QEQWtt_QEtQXttFn(Function):
    """dX = Q(E) Q(W^T)^T and dW = Q(E^T) Q(X^T)^T with a fresh sign vector per backward pass
    (backward.py:64-85 of the reference): the composition used when the layer's forward quantizers are not the
    fused production pair, so x and w arrive here as dense (already pseudo-quantized) tensors."""

    @staticmethod
    def forward(ctx, x, w, g_quantizer):
        ctx.save_for_backward(x, w)
        ctx.g = g_quantizer
        return torch.nn.functional.linear(x, w)

    @staticmethod
    def backward(ctx, e):
        x, w = ctx.saved_tensors
        g = ctx.g
        g.re_randomize()
        e2, x2 = _flat2d(e), _flat2d(x)
        if _packable(g, e2, x2, w):
            # four packed quantizations in the reference's order (E, W^T, E^T, X^T: one seed each), two MXFP4 GEMMs
            g._see(e2)
            alpha = (ops.SR_OPERAND_SCALE * g.out_scale) ** 2
            ec, es = g.pack(e2)
            wtc, wts = g.pack_t(w.contiguous())
            etc, ets = g.pack_t(e2)
            xtc, xts = g.pack_t(x2)
            dx = ops.gemm_mxfp4_tn(ec, es, wtc, wts, alpha, out_dtype=e2.dtype).reshape(x.shape)
            dw = ops.gemm_mxfp4_tn(etc, ets, xtc, xts, alpha, out_dtype=e2.dtype)
            return dx, dw, None
        qe, qwt = g(e2), g(w.t().contiguous())
        qet, qxt = g(e2.t().contiguous()), g(x2.t().contiguous())
        return (qe @ qwt.t()).reshape(x.shape), qet @ qxt.t(), None


class QEQWtt_QEtQXtt_Scheme(QEW_QEtX_Scheme):
    def forward(self, x, w):
        return QEQWtt_QEtQXttFn.apply(x, w, self.g_quantizer)


BACKWARD_SCHEMES = {
    "EW_EtX": EW_EtX_Scheme,
    "Q(E)W_Q(Et)X": QEW_QEtX_Scheme,
    "Q(E)Q(Wt)t_Q(Et)Q(Xt)t": QEQWtt_QEtQXtt_Scheme,
}
