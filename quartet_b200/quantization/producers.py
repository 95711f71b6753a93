"""A quantized linear layer together with the elementwise step that produces its input:

    rmsnorm_linear(x, norm_weight, eps, linear)   ==  linear(RMSNorm(x))              (llama.py:64-75, 124 / 113 of the reference)
    swiglu_linear(h, linear)                      ==  linear(silu(up) * gate)         (llama.py:112-114)

For the production combination of quantizers the forward quantizer reads the step's INPUT and applies the step
in registers, so the normalised / gated activation never exists in memory; the backward pass returns the
step's own gradient as well.  Any other combination, shape or device composes the step and the layer from
torch operations and the layer's ordinary forward.

The reference's model code calls the two steps separately; a model adopts the fused form by replacing
`self.c_attn(self.ln_1(x))`-style pairs with these calls (the harness model of this repository's tests does so
behind a flag).
"""
from __future__ import annotations

import torch

from .. import torch_ops


def _out_dtype(x: torch.Tensor, fallback: torch.dtype) -> torch.dtype:
    if torch.is_autocast_enabled():
        d = torch.get_autocast_dtype("cuda")
        return d if d == torch.bfloat16 else torch.float32
    return fallback


def _rmsnorm(x, weight, eps):
    return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)).type_as(x) * weight


def rmsnorm_linear(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, linear) -> torch.Tensor:
    if (norm_weight.dtype == torch.float32 and getattr(linear, "wgrad_sink", None) is None and linear._fusable(x)
            and x.shape[-1] == linear.in_features):
        # the norm's output is fp32 (an fp32 weight multiplies it), which is what the layer returns without autocast
        return torch.ops.quartet_b200.rmsnorm_linear_fwd(x, norm_weight, float(eps), linear.weight, linear._handle,
                                                         _out_dtype(x, torch.float32))[0]
    return linear(_rmsnorm(x, norm_weight, eps))


def swiglu_linear(h: torch.Tensor, linear) -> torch.Tensor:
    if getattr(linear, "wgrad_sink", None) is None and linear._fusable(h) and h.shape[-1] == 2 * linear.in_features:
        return torch.ops.quartet_b200.swiglu_linear_fwd(h, linear.weight, linear._handle, _out_dtype(h, h.dtype))[0]
    up, gate = h.split(h.shape[-1] // 2, dim=-1)
    return linear(torch.nn.functional.silu(up) * gate)
