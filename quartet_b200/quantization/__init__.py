"""Drop-in for the reference's `models.quantization` package (src/models/quantization/__init__.py):
exports QuantizedLinear, QUANTIZER_CLASSES and BACKWARD_SCHEMES with the same constructor and call
signatures, so model code that does

    from .quantization import QuantizedLinear, QUANTIZER_CLASSES, BACKWARD_SCHEMES

(src/models/llama.py:14, src/models/base.py:17) runs unchanged once `install()` has registered this
package under that module name.
"""
from __future__ import annotations

import sys

import torch
import torch.nn as nn

from .. import ops
from .backward import BACKWARD_SCHEMES, EW_EtX_Scheme, QEQWtt_QEtQXtt_Scheme
from .fused import QuartetLinearFn
from .quantizers import (AlbertTsengQuantizer, AlignedAlbertTsengQuantizer, BaseQuantizer, NoQuantizer,
                         QuestMXFP4Quantizer, mxfp4_forward_kernel_wrapper)

# Registry names of the reference that are not MXFP4 quantizers (research baselines built from
# plain torch ops, src/models/quantization/quantizers/{quest,baselines,adabin,noise}.py).  They are
# not on the accelerated path; asking for one says so instead of silently doing something else.
_OTHER_NAMES = (
    "NoiseQuantizer UniformQuantizer HalfHadamardUniformQuantizer STEQuantizer ClipQuantizer "
    "HalfHadamardClipQuantizer HadamardClipQuantizer TrustQuantizer HalfHadamardTrustQuantizer "
    "HadamardTrustQuantizer GaussianSTEQuantizer GaussianClipQuantizer GaussianTrustQuantizer "
    "HadamardGaussianClipQuantizer HalfHadamardGaussianTrustQuantizer HadamardGaussianTrustQuantizer "
    "FP4STEQuantizer FP4ClipQuantizer FP4TrustQuantizer HalfHadamardFP4ClipQuantizer HadamardFP4ClipQuantizer "
    "HalfHadamardFP4TrustQuantizer HadamardFP4TrustQuantizer FourEightMaskedQuantizer FourEightSTEQuantizer "
    "FourEightClipQuantizer FourEightTrustQuantizer HalfHadamardFourEightTrustQuantizer "
    "HalfHadamardTwoFourTrustQuantizer HadamardFourEightTrustQuantizer PACTQuantizer LSQQuantizer "
    "LSQPlusActivationQuantizer LSQPlusWeightQuantizer AdaBinWeightQuantizer AdaBinActivationQuantizer"
).split()


def _not_built(name):
    def ctor(*a, **k):
        raise NotImplementedError(
            f"{name} is a plain-torch research baseline of the reference and is outside the MXFP4 path this "
            "library accelerates; use the reference's own class for it"
        )

    ctor.__name__ = name
    return ctor


QUANTIZER_CLASSES = {name: _not_built(name) for name in _OTHER_NAMES}
QUANTIZER_CLASSES.update(
    {
        "NoQuantizer": NoQuantizer,
        "AlbertTsengQuantizer": AlbertTsengQuantizer,
        "QuestMXFP4Quantizer": QuestMXFP4Quantizer,
        "AlignedAlbertTsengQuantizer": AlignedAlbertTsengQuantizer,
    }
)


class QuantizedLinear(nn.Linear):
    """src/models/quantization/__init__.py:11-42, same constructor and forward.

    When the three quantizers and the scheme are the production combination, forward/backward run
    as one fused autograd function on packed MXFP4 operands; any other combination composes the
    modules exactly like the reference does."""

    def __init__(self, in_features, out_features, weight_quantizer=None, activation_quantizer=None,
                 gradient_quantizer=None, backward_scheme=None, **kwargs):
        super().__init__(in_features, out_features, **kwargs)
        if weight_quantizer is None:
            weight_quantizer = NoQuantizer()
        if activation_quantizer is None:
            activation_quantizer = NoQuantizer()
        if gradient_quantizer is None:
            gradient_quantizer = NoQuantizer()
        if backward_scheme is None:
            backward_scheme = EW_EtX_Scheme()
        self.weight_quantizer = weight_quantizer
        self.activation_quantizer = activation_quantizer
        self.backward_scheme = backward_scheme
        self.backward_scheme.g_quantizer = gradient_quantizer

    def _fusable(self, x) -> bool:
        g = self.backward_scheme.g_quantizer
        return (
            type(self.weight_quantizer) is QuestMXFP4Quantizer
            and type(self.activation_quantizer) is QuestMXFP4Quantizer
            and type(g) in (AlbertTsengQuantizer, AlignedAlbertTsengQuantizer)
            and type(self.backward_scheme) is QEQWtt_QEtQXtt_Scheme
            and g.rerotate in (None, "signs")
            and self.bias is None
            and x.is_cuda
            and self.in_features % 128 == 0
            and self.out_features % 128 == 0
            and x.dtype in (torch.bfloat16, torch.float32)
        )

    def export_mxfp4(self):
        """The forward-quantized weight as real MXFP4: (codes uint8 [N, K/2], scales E8M0 uint8 in the
        blocked 128 x 4 layout, had_scale).  The values are in the rotated basis (groups of 32 along K
        multiplied by the forward Hadamard matrix), i.e. exactly the B operand of the forward GEMM --
        the layout a block-scaled MXFP4 inference GEMM consumes (`to_blocked`,
        notebooks/benchmark_mxfp4.ipynb:1015-1016 of the reference); the reference itself only
        checkpoints fp32 weights (src/optim/utils.py:245-256)."""
        wq = self.weight_quantizer
        if type(wq) is not QuestMXFP4Quantizer or not self.weight.is_cuda:
            raise RuntimeError("export_mxfp4 needs a QuestMXFP4Quantizer weight quantizer and a CUDA weight")
        wq._see(self.weight)
        if wq._sign_word() != 0:
            raise RuntimeError("the forward rotation carries a sign vector; only the plain Hadamard rotation is exported")
        with torch.no_grad():
            codes, sf, _ = ops.quant_fwd(self.weight.detach().contiguous(), wq.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=False)
        return codes, sf, wq.had_scale

    def forward(self, x):
        if self._fusable(x):
            aq, wq = self.activation_quantizer, self.weight_quantizer
            aq._see(x)
            wq._see(self.weight)
            if aq._sign_word() == 0 and wq._sign_word() == 0:
                if torch.is_autocast_enabled():
                    out_dtype = torch.get_autocast_dtype("cuda")
                    if out_dtype != torch.bfloat16:
                        out_dtype = torch.float32
                else:
                    out_dtype = x.dtype
                return QuartetLinearFn.apply(x, self.weight, aq, wq, self.backward_scheme.g_quantizer, out_dtype,
                                             getattr(self, "wgrad_sink", None))
        xq = self.activation_quantizer(x)
        wq = self.weight_quantizer(self.weight)
        return self.backward_scheme(xq, wq)


def install(module_name: str = "models.quantization") -> None:
    """Register this package under the name the reference's model code imports."""
    me = sys.modules[__name__]
    sys.modules[module_name] = me
    sys.modules[module_name + ".quantizers"] = sys.modules[__name__ + ".quantizers"]
    sys.modules[module_name + ".backward"] = sys.modules[__name__ + ".backward"]
    parent = module_name.rsplit(".", 1)[0]
    if parent in sys.modules:
        setattr(sys.modules[parent], module_name.rsplit(".", 1)[1], me)
