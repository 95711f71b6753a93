"""Host-side mirror of the reference's MXFP4 quantizer modules
(src/models/quantization/quantizers/{base,mxfp4,mxfp4_triton}.py): same class names, constructor
keywords, attributes and forward/backward meaning, computed by the sm_100a kernels.

Stand-alone use (`quantizer(x)`) returns the pseudo-quantized tensor like the reference does
(quantize, then de-quantize, same dtype and shape); QuantizedLinear short-cuts the production
combination into one fused real-MXFP4 path (see fused.py).
"""
from __future__ import annotations

import random

import torch
import torch.nn as nn

from .. import ops


def _sylvester32() -> torch.Tensor:
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < 32:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h


def decompose_rotation(hm: torch.Tensor):
    """A 32x32 matrix of the form scale * Sylvester @ diag(s) -> (scale, sign word).

    Raises NotImplementedError for anything else (the reference's rerotate="O32" draws a dense
    random orthogonal matrix, mxfp4.py:61-64; a dense-rotation kernel is not built)."""
    if hm.shape != (32, 32):
        raise NotImplementedError("only hadamard_dim=32 is built")
    m = hm.detach().to("cpu", torch.float64)
    scale = float(m[0, 0].abs())
    s = torch.sign(m[0])
    if scale == 0 or not torch.equal(torch.sign(m), torch.sign(_sylvester32() * s[None, :])) or not torch.allclose(m.abs(), torch.full_like(m, scale)):
        raise NotImplementedError("rotation is not a sign-flipped Sylvester-Hadamard matrix (rerotate='O32' is not built)")
    word = 0
    for j in range(32):
        if s[j] < 0:
            word |= 1 << j
    return scale, word


def _as_rows(x: torch.Tensor) -> torch.Tensor:
    """The reference kernel sees a flat tensor in groups of 32; the kernels here want [rows, cols % 128 == 0]."""
    x = x.contiguous()
    if x.dim() >= 2 and x.shape[-1] % 128 == 0:
        return x.reshape(-1, x.shape[-1])
    if x.numel() % 128 != 0:
        raise ValueError(f"number of elements ({x.numel()}) must be a multiple of 128")
    return x.reshape(-1, 128)


@torch.compiler.disable()
def mxfp4_forward_kernel_wrapper(x, hadamard_matrix, return_clip_mask=False, gaussian_scale=3 / 4, stochastic_round=False,
                                 quest=True):
    """Same signature and result as the reference's wrapper (mxfp4_triton.py:177-220): the rotated,
    quantized and de-quantized tensor in x's dtype, plus an optional bool clip mask.  Stochastic
    rounding draws `random.randint(0, 1000000)` like the reference and replays tl.rand(seed, offset),
    so equal Python RNG state gives equal output."""
    scale, signs = decompose_rotation(hadamard_matrix)
    x2 = _as_rows(x)
    if quest:
        if stochastic_round:
            raise NotImplementedError("quest=True with stochastic rounding is not used by any quantizer module")
        if signs:
            raise NotImplementedError("sign-flipped rotation in the forward (std-scaled) quantizer is not built")
        codes, sf, mask = ops.quant_fwd(x2, scale, gaussian_scale, return_mask=return_clip_mask)
        out = ops.dequant(codes, sf, 1.0, x.dtype).reshape(x.shape)
        return out, (ops.unpack_mask(mask).reshape(x.shape) if return_clip_mask else None)
    if stochastic_round:
        seed = random.randint(0, 1000000)
        codes, sf = ops.quant_bwd(x2, scale, signs=signs, rounding=ops.ROUND_SR_TLRAND, seed=seed)
    else:
        codes, sf = ops.quant_bwd(x2, scale, signs=signs, rounding=ops.ROUND_NEAREST)
    out = ops.dequant(codes, sf, ops.SR_OPERAND_SCALE, x.dtype).reshape(x.shape)
    mask = None
    if return_clip_mask:  # |v| < 6 always holds under absmax scaling
        mask = torch.ones_like(x, dtype=torch.bool)
    return out, mask


class BaseQuantizer(nn.Module):
    """src/models/quantization/quantizers/base.py:6-16"""

    def __init__(self, bits=4):
        super().__init__()
        self.bits = bits
        self.n_levels = 2 ** bits

    def forward(self, x):
        raise NotImplementedError

    def re_randomize(self):
        pass


class NoQuantizer(BaseQuantizer):
    """base.py:19-24"""

    def __init__(self, **kwargs):
        super().__init__(16)

    def forward(self, x):
        return x


class _Rotation32(BaseQuantizer):
    """State shared by the three MXFP4 quantizers: a 32x32 rotation kept as (entry magnitude, sign word).

    `hadamard_matrix` is materialised on demand so code that reads or assigns the attribute keeps
    working (mxfp4.py:42-50); like the reference, the matrix takes the dtype of the last input seen
    (the cast at mxfp4.py:49 is sticky) and the sign vector accumulates over re_randomize() calls.
    The sign word lives on the device so re-randomising never synchronises with the host.
    """

    def __init__(self, hadamard_dim=32, rerotate=None):
        super().__init__(4)
        if hadamard_dim != 32:
            raise NotImplementedError("only hadamard_dim=32 is built")
        if rerotate not in (None, "signs", "O32"):
            raise ValueError(f"Invalid rerotate value: {rerotate}")
        self.hadamard_dim = hadamard_dim
        self.rerotate = rerotate
        self._h_dtype = torch.float32
        self._signs_host = 0          # valid while _signs_dev is None
        self._signs_dev = None        # int64[1] on the compute device once re_randomize() ran there

    # -- rotation state --
    @property
    def had_scale(self) -> float:
        return float(torch.tensor(32 ** -0.5, dtype=torch.float32).to(self._h_dtype))

    def _sign_word(self) -> int:
        if self._signs_dev is not None:
            return int(self._signs_dev.item()) & 0xFFFFFFFF
        return self._signs_host

    @property
    def hadamard_matrix(self) -> torch.Tensor:
        word = self._sign_word()
        s = torch.tensor([-1.0 if (word >> j) & 1 else 1.0 for j in range(32)], dtype=torch.float64)
        dev = self._signs_dev.device if self._signs_dev is not None else "cpu"
        return (_sylvester32() * s[None, :] * self.had_scale).to(self._h_dtype).to(dev)

    @hadamard_matrix.setter
    def hadamard_matrix(self, hm: torch.Tensor):
        scale, word = decompose_rotation(hm)
        self._h_dtype = hm.dtype
        if abs(scale - self.had_scale) > 1e-6:
            raise NotImplementedError("rotation entries must be +-32**-0.5 in the matrix dtype")
        self._signs_host, self._signs_dev = word, None

    def _see(self, x: torch.Tensor):
        # mxfp4.py:49 / :160: self.hadamard_matrix = self.hadamard_matrix.to(x.device).to(x.dtype)
        self._h_dtype = x.dtype
        if self._signs_dev is not None and self._signs_dev.device != x.device:
            self._signs_dev = self._signs_dev.to(x.device)

    def re_randomize(self, device=None):
        """mxfp4.py:52-68: 'signs' multiplies the columns of H by fresh random signs (same
        torch.randint call on the same device, so the global RNG advances identically)."""
        if self.rerotate is None:
            return
        if self.rerotate == "O32":
            raise NotImplementedError("rerotate='O32' (dense random orthogonal rotation) is not built")
        dev = device or (self._signs_dev.device if self._signs_dev is not None else "cuda")
        draw = torch.randint(0, 2, (32,), device=dev, dtype=self._h_dtype) * 2 - 1
        bits = ((draw < 0).to(torch.int64) << torch.arange(32, device=dev, dtype=torch.int64)).sum().reshape(1)
        if self._signs_dev is None:
            self._signs_dev = torch.full((1,), self._signs_host, dtype=torch.int64, device=dev)
        self._signs_dev = self._signs_dev ^ bits

    def sign_args(self):
        """kwargs for the ops: the sign word either as an immediate or as a device pointer."""
        if self._signs_dev is not None:
            return {"signs": 0, "signs_dev": self._signs_dev}
        return {"signs": self._signs_host, "signs_dev": None}


class _QuestFn(torch.autograd.Function):
    """QuestMXFP4QuantizerFn (mxfp4.py:127-146)."""

    @staticmethod
    def forward(ctx, x, had_scale):
        x2 = _as_rows(x)
        codes, sf, mask = ops.quant_fwd(x2, had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=True)
        ctx.save_for_backward(mask)
        ctx.had_scale, ctx.x_shape = had_scale, x.shape
        return ops.dequant(codes, sf, 1.0, x.dtype).reshape(x.shape)

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        g2 = grad_output.contiguous().reshape(mask.shape[0], -1)
        return ops.unrotate_mask(g2, mask, ctx.had_scale).reshape(ctx.x_shape), None


class QuestMXFP4Quantizer(_Rotation32):
    """Forward quantizer module (mxfp4.py:149-179): std-scaled round-to-nearest with a clip mask."""

    def forward(self, x):
        self._see(x)
        if self._sign_word():
            raise NotImplementedError("sign-flipped rotation in the forward (std-scaled) quantizer is not built")
        return _QuestFn.apply(x, self.had_scale)


class _AbsmaxFn(torch.autograd.Function):
    """AlbertTsengQuantizerFn / AlignedAlbertTsengQuantizerFn (mxfp4.py:15-34, 71-92)."""

    @staticmethod
    def forward(ctx, x, q, stochastic, out_scale):
        x2 = _as_rows(x)
        if stochastic:
            seed = random.randint(0, 1000000)  # mxfp4_triton.py:196-197
            codes, sf = ops.quant_bwd(x2, q.had_scale, rounding=q.sr_rounding, seed=seed, **q.sign_args())
        else:
            codes, sf = ops.quant_bwd(x2, q.had_scale, rounding=ops.ROUND_NEAREST, **q.sign_args())
        ctx.q, ctx.x_shape = q, x.shape
        return ops.dequant(codes, sf, ops.SR_OPERAND_SCALE * out_scale, x.dtype).reshape(x.shape)

    @staticmethod
    def backward(ctx, grad_output):
        q = ctx.q
        # grad @ (H diag(s))^T = (grad * s) @ H^T
        word = q._sign_word()
        g = grad_output.contiguous().reshape(-1, 32)
        if word:
            s = torch.tensor([-1.0 if (word >> j) & 1 else 1.0 for j in range(32)], dtype=g.dtype, device=g.device)
            g = g * s
        return ops.unrotate_mask(g, None, q.had_scale).reshape(ctx.x_shape), None, None, None


class AlbertTsengQuantizer(_Rotation32):
    """Backward (gradient) quantizer module (mxfp4.py:37-68): absmax scale, stochastic rounding.

    `sr_rounding` selects the noise source of stand-alone and fused calls: the library's own Philox
    dither stream (default) or ops.ROUND_SR_TLRAND to replay the reference's tl.rand stream."""

    def __init__(self, hadamard_dim=32, stochastic=True, rerotate=None):
        super().__init__(hadamard_dim, rerotate)
        self.stochastic = stochastic
        self.sr_rounding = ops.ROUND_SR_PHILOX
        self.out_scale = 1.0

    def forward(self, x):
        self._see(x)
        return _AbsmaxFn.apply(x, self, self.stochastic, self.out_scale)


class AlignedAlbertTsengQuantizer(_Rotation32):
    """mxfp4.py:95-124: round-to-nearest absmax quantizer whose output is multiplied by 1.009276."""

    def __init__(self, hadamard_dim=32, rerotate=None):
        super().__init__(hadamard_dim, rerotate)
        self.stochastic = False
        self.sr_rounding = ops.ROUND_NEAREST
        self.out_scale = 1.009276

    def forward(self, x):
        self._see(x)
        return _AbsmaxFn.apply(x, self, False, self.out_scale)
