"""Host-side mirror of the reference's MXFP4 quantizer modules
(src/models/quantization/quantizers/{base,mxfp4,mxfp4_triton}.py): same class names, constructor
keywords, attributes and forward/backward meaning, computed by the sm_100a kernels.

Stand-alone use (`quantizer(x)`) returns the pseudo-quantized tensor like the reference does
(quantize, then de-quantize, same dtype and shape); QuantizedLinear short-cuts the production
combination into one fused real-MXFP4 path (fused.py / torch_ops.py).

Rotations.  The kernels have the 32-point Sylvester-Hadamard rotation built in, with an optional sign
vector (H @ diag(s), what rerotate="signs" produces); a quantizer in that state keeps only the entry
magnitude and a 32-bit sign word.  Any other rotation -- hadamard_dim 64 or 128
(sweep_tokens_backward.sh:52-53 of the reference passes it as a keyword), the dense random orthogonal
matrix of rerotate="O32" (mxfp4.py:61-64), or a matrix assigned to `hadamard_matrix` -- is kept as a dense
matrix: the rotation then is a torch matmul and the rotation-free kernel entry (`quant_group32`) does the
scaling, rounding and packing.
"""
from __future__ import annotations

import random

import torch
import torch.nn as nn

from .. import ops


def _sylvester(n: int) -> torch.Tensor:
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h


def decompose_rotation(hm: torch.Tensor):
    """A 32x32 matrix of the form scale * Sylvester @ diag(s) -> (scale, sign word); None for anything else."""
    if hm.shape != (32, 32):
        return None
    m = hm.detach().to("cpu", torch.float64)
    scale = float(m[0, 0].abs())
    s = torch.sign(m[0])
    if scale == 0 or not torch.equal(torch.sign(m), torch.sign(_sylvester(32) * s[None, :])) or not torch.allclose(m.abs(), torch.full_like(m, scale)):
        return None
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


def _rotate_dense(x2: torch.Tensor, hm: torch.Tensor) -> torch.Tensor:
    """`x.view(-1, d) @ H` with both operands in x's dtype and fp32 accumulation, as fp32 [rows, cols]
    (mxfp4_triton.py:45-47: tl.dot returns fp32)."""
    d = hm.shape[-1]
    h = hm.to(x2.device).to(x2.dtype).float()
    return (x2.float().reshape(-1, d) @ h).reshape(x2.shape)


@torch.compiler.disable()
def mxfp4_forward_kernel_wrapper(x, hadamard_matrix, return_clip_mask=False, gaussian_scale=3 / 4, stochastic_round=False,
                                 quest=True):
    """Same signature and result as the reference's wrapper (mxfp4_triton.py:177-220): the rotated,
    quantized and de-quantized tensor in x's dtype, plus an optional bool clip mask.  Stochastic
    rounding draws `random.randint(0, 1000000)` like the reference and replays tl.rand(seed, offset),
    so equal Python RNG state gives equal output."""
    if quest and stochastic_round:
        raise NotImplementedError("quest=True with stochastic rounding is not used by any quantizer module")
    x2 = _as_rows(x)
    fast = decompose_rotation(hadamard_matrix)
    if fast is not None and not (quest and fast[1]):
        scale, signs = fast
        if quest:
            codes, sf, mask = ops.quant_fwd(x2, scale, gaussian_scale, return_mask=return_clip_mask)
        elif stochastic_round:
            codes, sf = ops.quant_bwd(x2, scale, signs=signs, rounding=ops.ROUND_SR_TLRAND, seed=random.randint(0, 1000000))
        else:
            codes, sf = ops.quant_bwd(x2, scale, signs=signs, rounding=ops.ROUND_NEAREST)
    else:  # any other rotation: dense matmul here, rotation-free scaling / rounding / packing in the kernel
        xh = _rotate_dense(x2, hadamard_matrix)
        if quest:
            codes, sf, mask = ops.quant_group32(xh, 0, gaussian_scale, return_mask=return_clip_mask)
        elif stochastic_round:
            codes, sf, _ = ops.quant_group32(xh, 1, rounding=ops.ROUND_SR_TLRAND, seed=random.randint(0, 1000000))
        else:
            codes, sf, _ = ops.quant_group32(xh, 1, rounding=ops.ROUND_NEAREST)
    if quest:
        out = ops.dequant(codes, sf, 1.0, x.dtype).reshape(x.shape)
        return out, (ops.unpack_mask(mask).reshape(x.shape) if return_clip_mask else None)
    out = ops.dequant(codes, sf, ops.SR_OPERAND_SCALE, x.dtype).reshape(x.shape)
    # |v| < 6 always holds under absmax scaling
    return out, (torch.ones_like(x, dtype=torch.bool) if return_clip_mask else None)


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


class _Rotation(BaseQuantizer):
    """State shared by the three MXFP4 quantizers: the rotation, kept as (entry magnitude, sign word) while it
    is a sign-flipped 32-point Sylvester matrix and as a dense matrix otherwise.

    `hadamard_matrix` is materialised on demand so code that reads or assigns the attribute keeps
    working (mxfp4.py:42-50); like the reference, the matrix takes the dtype of the last input seen
    (the cast at mxfp4.py:49 is sticky) and the sign vector accumulates over re_randomize() calls.
    The sign word lives on the device so re-randomising never synchronises with the host.
    """

    def __init__(self, hadamard_dim=32, rerotate=None):
        super().__init__(4)
        if hadamard_dim < 32 or hadamard_dim & (hadamard_dim - 1) or hadamard_dim % 32:
            raise ValueError(f"hadamard_dim must be a power of two >= 32 (scale groups are 32 wide), got {hadamard_dim}")
        if rerotate not in (None, "signs", "O32"):
            raise ValueError(f"Invalid rerotate value: {rerotate}")
        self.hadamard_dim = hadamard_dim
        self.rerotate = rerotate
        self._h_dtype = torch.float32
        self._signs_host = 0          # valid while _signs_dev is None
        self._signs_dev = None        # int64[1] on the compute device once re_randomize() ran there
        self._dense = None            # fp32 [d, d] when the rotation is not a sign-flipped Sylvester-32 matrix
        if hadamard_dim != 32:
            self._dense = (_sylvester(hadamard_dim) * hadamard_dim ** -0.5).float()

    # -- rotation state --
    @property
    def is_builtin_rotation(self) -> bool:
        return self._dense is None

    @property
    def had_scale(self) -> float:
        return float(torch.tensor(32 ** -0.5, dtype=torch.float32).to(self._h_dtype))

    def _sign_word(self) -> int:
        if self._signs_dev is not None:
            return int(self._signs_dev.item()) & 0xFFFFFFFF
        return self._signs_host

    @property
    def hadamard_matrix(self) -> torch.Tensor:
        if self._dense is not None:
            return self._dense.to(self._h_dtype)
        word = self._sign_word()
        s = torch.tensor([-1.0 if (word >> j) & 1 else 1.0 for j in range(32)], dtype=torch.float64)
        dev = self._signs_dev.device if self._signs_dev is not None else "cpu"
        return (_sylvester(32) * s[None, :] * self.had_scale).to(self._h_dtype).to(dev)

    @hadamard_matrix.setter
    def hadamard_matrix(self, hm: torch.Tensor):
        if hm.dim() != 2 or hm.shape[0] != hm.shape[1] or hm.shape[0] % 32:
            raise ValueError("the rotation must be a square matrix whose size is a multiple of 32")
        self._h_dtype = hm.dtype
        self.hadamard_dim = hm.shape[0]
        fast = decompose_rotation(hm)
        if fast is not None and abs(fast[0] - self.had_scale) <= 1e-6:
            self._signs_host, self._signs_dev, self._dense = fast[1], None, None
        else:
            self._dense = hm.detach().float()

    def _see(self, x: torch.Tensor):
        # mxfp4.py:49 / :160: self.hadamard_matrix = self.hadamard_matrix.to(x.device).to(x.dtype)
        if self._dense is not None and self._h_dtype != x.dtype:
            self._dense = self._dense.to(x.dtype).float()  # the reference's cast rounds the stored matrix for good
        self._h_dtype = x.dtype
        if self._signs_dev is not None and self._signs_dev.device != x.device:
            self._signs_dev = self._signs_dev.to(x.device)
        if self._dense is not None and self._dense.device != x.device:
            self._dense = self._dense.to(x.device)

    def re_randomize(self, device=None):
        """mxfp4.py:52-68.  'signs' multiplies the columns of H by fresh random signs (same torch.randint call on
        the same device, so the global RNG advances identically); 'O32' draws a random orthogonal matrix (the
        orthogonal factor of a Gaussian matrix; computed in fp32 whatever the matrix dtype, where the reference's
        own bf16 SVD call fails)."""
        if self.rerotate is None:
            return
        d = self.hadamard_dim
        if self._dense is not None:
            dev = device or self._dense.device
        else:
            dev = device or (self._signs_dev.device if self._signs_dev is not None else "cuda")
        if self.rerotate == "O32":
            gauss = torch.randn(d, d, device=dev, dtype=torch.float32)
            u, _, vh = torch.linalg.svd(gauss)
            self._dense = (u @ vh).to(self._h_dtype).float()
            self._signs_host, self._signs_dev = 0, None
            return
        draw = torch.randint(0, 2, (d,), device=dev, dtype=self._h_dtype)  # the reference's call; its signs are 2 * draw - 1
        if self._dense is not None:
            self._dense = self._dense.to(dev) * (draw.float() * 2 - 1)[None, :]
            return
        if self._signs_dev is None or self._signs_dev.device != draw.device:
            self._signs_dev = torch.full((1,), self._signs_host if self._signs_dev is None else self._sign_word(), dtype=torch.int64, device=dev)
        if draw.is_cuda and draw.dtype in (torch.bfloat16, torch.float32):
            ops.fold_signs(draw, self._signs_dev)  # one launch: pack the 32 signs and fold them into the device word
        else:
            bits = ((draw == 0).to(torch.int64) << torch.arange(32, device=dev, dtype=torch.int64)).sum().reshape(1)
            self._signs_dev = self._signs_dev ^ bits

    def sign_args(self):
        """kwargs for the ops: the sign word either as an immediate or as a device pointer."""
        if self._signs_dev is not None:
            return {"signs": 0, "signs_dev": self._signs_dev}
        return {"signs": self._signs_host, "signs_dev": None}

    def _unrotate(self, g2: torch.Tensor, mask) -> torch.Tensor:
        """(g * mask).view(-1, d) @ H^T  (mxfp4.py:30-34, 142-146)."""
        if self._dense is not None:
            if mask is not None:
                g2 = g2 * ops.unpack_mask(mask).reshape(g2.shape).to(g2.dtype)
            d = self.hadamard_dim
            h = self._dense.to(g2.device).to(g2.dtype)
            return (g2.reshape(-1, d) @ h.t()).reshape(g2.shape)
        word = self._sign_word()
        if word:  # grad @ (H diag(s))^T = (grad * s) @ H^T
            s = torch.tensor([-1.0 if (word >> j) & 1 else 1.0 for j in range(32)], dtype=g2.dtype, device=g2.device)
            g2 = (g2.reshape(-1, 32) * s).reshape(g2.shape)
            if mask is not None:
                raise NotImplementedError("a clip mask together with a sign-flipped rotation")
        return ops.unrotate_mask(g2.contiguous(), mask, self.had_scale)


class _QuestFn(torch.autograd.Function):
    """QuestMXFP4QuantizerFn (mxfp4.py:127-146)."""

    @staticmethod
    def forward(ctx, x, q):
        x2 = _as_rows(x)
        if q.is_builtin_rotation and q._sign_word() == 0:
            codes, sf, mask = ops.quant_fwd(x2, q.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=True)
        else:
            codes, sf, mask = ops.quant_group32(_rotate_dense(x2, q.hadamard_matrix), 0, ops.QUEST_GAUSSIAN_SCALE)
        ctx.save_for_backward(mask)
        ctx.q, ctx.x_shape = q, x.shape
        return ops.dequant(codes, sf, 1.0, x.dtype).reshape(x.shape)

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        q = ctx.q
        g2 = grad_output.contiguous().reshape(mask.shape[0], -1)
        if q.is_builtin_rotation and q._sign_word() == 0:
            return ops.unrotate_mask(g2, mask, q.had_scale).reshape(ctx.x_shape), None
        h = q.hadamard_matrix.to(g2.device).to(g2.dtype)
        g2 = g2 * ops.unpack_mask(mask).reshape(g2.shape).to(g2.dtype)
        return (g2.reshape(-1, h.shape[0]) @ h.t()).reshape(ctx.x_shape), None


class QuestMXFP4Quantizer(_Rotation):
    """Forward quantizer module (mxfp4.py:149-179): std-scaled round-to-nearest with a clip mask."""

    def forward(self, x):
        self._see(x)
        return _QuestFn.apply(x, self)


class _AbsmaxFn(torch.autograd.Function):
    """AlbertTsengQuantizerFn / AlignedAlbertTsengQuantizerFn (mxfp4.py:15-34, 71-92)."""

    @staticmethod
    def forward(ctx, x, q):
        codes, sf = q.pack(_as_rows(x))
        ctx.q, ctx.x_shape = q, x.shape
        out = ops.dequant(codes, sf, ops.SR_OPERAND_SCALE, x.dtype).reshape(x.shape)
        if q.out_scale != 1.0:
            out *= q.out_scale  # applied to the stored tensor, in its dtype, like `x_dequantized *= 1.009276` (mxfp4.py:82)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        g2 = grad_output.contiguous().reshape(-1, ctx.q.hadamard_dim)
        return ctx.q._unrotate(g2, None).reshape(ctx.x_shape), None


class AbsmaxRotation32(_Rotation):
    """Common part of the two absmax-scaled (gradient) quantizers: packed MXFP4 output through the kernels."""

    stochastic = True
    sr_rounding = ops.ROUND_SR_PHILOX
    out_scale = 1.0

    def _rounding_and_seed(self):
        if self.stochastic:
            return self.sr_rounding, random.randint(0, 1000000)  # one draw per quantizer call, mxfp4_triton.py:196-197
        return ops.ROUND_NEAREST, 0

    def pack(self, x2: torch.Tensor):
        """[rows, cols] -> (codes [rows, cols/2], blocked scales): groups along cols."""
        rounding, seed = self._rounding_and_seed()
        if self.is_builtin_rotation:
            return ops.quant_bwd(x2, self.had_scale, rounding=rounding, seed=seed, **self.sign_args())
        codes, sf, _ = ops.quant_group32(_rotate_dense(x2, self.hadamard_matrix), 1, rounding=rounding, seed=seed)
        return codes, sf

    def pack_t(self, x2: torch.Tensor):
        """[rows, cols] -> MXFP4 of the TRANSPOSE (codes [cols, rows/2], blocked scales): groups along rows of x2,
        without materialising the transpose when the rotation is the built-in one."""
        if self.is_builtin_rotation:
            rounding, seed = self._rounding_and_seed()
            return ops.quant_bwd_t(x2, self.had_scale, rounding=rounding, seed=seed, **self.sign_args())
        return self.pack(x2.t().contiguous())

    def forward(self, x):
        self._see(x)
        return _AbsmaxFn.apply(x, self)


class AlbertTsengQuantizer(AbsmaxRotation32):
    """Backward (gradient) quantizer module (mxfp4.py:37-68): absmax scale, stochastic rounding.

    `sr_rounding` selects the noise source of stand-alone and fused calls: the library's own Philox
    dither stream (default) or ops.ROUND_SR_TLRAND to replay the reference's tl.rand stream."""

    def __init__(self, hadamard_dim=32, stochastic=True, rerotate=None):
        super().__init__(hadamard_dim, rerotate)
        self.stochastic = stochastic
        self.sr_rounding = ops.ROUND_SR_PHILOX
        self.out_scale = 1.0


class AlignedAlbertTsengQuantizer(AbsmaxRotation32):
    """mxfp4.py:95-124: round-to-nearest absmax quantizer whose output is multiplied by 1.009276."""

    def __init__(self, hadamard_dim=32, rerotate=None):
        super().__init__(hadamard_dim, rerotate)
        self.stochastic = False
        self.sr_rounding = ops.ROUND_NEAREST
        self.out_scale = 1.009276
