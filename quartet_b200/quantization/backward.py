"""Backward schemes, same names and behaviour as src/models/quantization/backward.py."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.autograd import Function


class EW_EtX_Scheme(nn.Module):
    """backward.py:11-17"""

    def __init__(self):
        super().__init__()
        self.g_quantizer = None

    def forward(self, x, w):
        return F.linear(x, w, None)


class QEW_QEtXFn(Function):
    """backward.py:21-45"""

    @staticmethod
    def forward(ctx, x, w, g_quantizer):
        ctx.save_for_backward(x, w)
        ctx.g_quantizer = g_quantizer
        return F.linear(x, w, None)

    @staticmethod
    def backward(ctx, e):
        x, w = ctx.saved_tensors
        grad_x = F.linear(ctx.g_quantizer(e), w.T, None)
        m = math.prod(x.shape[:-1])
        grad_w = torch.einsum("ib,bj->ij", ctx.g_quantizer(e.reshape(m, -1).T.contiguous()), x.reshape(m, -1))
        return grad_x, grad_w, None


class QEW_QEtX_Scheme(EW_EtX_Scheme):
    def forward(self, x, w):
        return QEW_QEtXFn.apply(x, w, self.g_quantizer)


class QEQWtt_QEtQXttFn(Function):
    """backward.py:57-85, un-fused: used when the quantizer combination is not the production one."""

    @staticmethod
    def forward(ctx, x, w, g_quantizer):
        ctx.save_for_backward(x, w)
        ctx.g_quantizer = g_quantizer
        return F.linear(x, w, None)

    @staticmethod
    def backward(ctx, e):
        x, w = ctx.saved_tensors
        ctx.g_quantizer.re_randomize()
        grad_x = F.linear(ctx.g_quantizer(e), ctx.g_quantizer(w.T.contiguous()), None)
        m = math.prod(x.shape[:-1])
        grad_w = torch.einsum(
            "ib,jb->ij",
            ctx.g_quantizer(e.reshape(m, -1).T.contiguous()),
            ctx.g_quantizer(x.reshape(m, -1).T.contiguous()),
        )
        return grad_x, grad_w, None


class QEQWtt_QEtQXtt_Scheme(QEW_QEtX_Scheme):
    def forward(self, x, w):
        return QEQWtt_QEtQXttFn.apply(x, w, self.g_quantizer)


BACKWARD_SCHEMES = {
    "EW_EtX": EW_EtX_Scheme,
    "Q(E)W_Q(Et)X": QEW_QEtX_Scheme,
    "Q(E)Q(Wt)t_Q(Et)Q(Xt)t": QEQWtt_QEtQXtt_Scheme,
}
