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

from .. import ops, torch_ops
from .backward import BACKWARD_SCHEMES, EW_EtX_Scheme, QEQWtt_QEtQXtt_Scheme
from .fused import QuartetLinearFn
from .producers import rmsnorm_linear, swiglu_linear  # noqa: F401
from .quantizers import (AbsmaxRotation32, AlbertTsengQuantizer, AlignedAlbertTsengQuantizer, BaseQuantizer, NoQuantizer,
                         QuestMXFP4Quantizer, mxfp4_forward_kernel_wrapper)

# Registry names of the reference that are not MXFP4 quantizers (research baselines built from plain torch
# ops): name -> file of src/models/quantization/quantizers/ that defines the class.  They are not on the
# accelerated path.  Asking for one builds the REFERENCE'S OWN class, imported from a reference checkout named
# by the environment variable QUARTET_REF (its `src` directory), so that ablations such as
# `--w-quant NoiseQuantizer` keep running next to the accelerated path; without a checkout it raises.
_OTHER_NAMES = {
    "noise": "NoiseQuantizer",
    "baselines": "UniformQuantizer PACTQuantizer LSQQuantizer LSQPlusActivationQuantizer LSQPlusWeightQuantizer",
    "adabin": "AdaBinWeightQuantizer AdaBinActivationQuantizer",
    "quest": (
        "HalfHadamardUniformQuantizer STEQuantizer ClipQuantizer HalfHadamardClipQuantizer HadamardClipQuantizer "
        "TrustQuantizer HalfHadamardTrustQuantizer HadamardTrustQuantizer GaussianSTEQuantizer GaussianClipQuantizer "
        "GaussianTrustQuantizer HadamardGaussianClipQuantizer HalfHadamardGaussianTrustQuantizer HadamardGaussianTrustQuantizer "
        "FP4STEQuantizer FP4ClipQuantizer FP4TrustQuantizer HalfHadamardFP4ClipQuantizer HadamardFP4ClipQuantizer "
        "HalfHadamardFP4TrustQuantizer HadamardFP4TrustQuantizer FourEightMaskedQuantizer FourEightSTEQuantizer "
        "FourEightClipQuantizer FourEightTrustQuantizer HalfHadamardFourEightTrustQuantizer "
        "HalfHadamardTwoFourTrustQuantizer HadamardFourEightTrustQuantizer"
    ),
}
_REF_PACKAGE = "quartet_reference_quantizers"


def _reference_module(stem: str):
    """Imports one file of the reference's quantizers directory under a private package name (its own
    `__init__` is not run, so nothing else of the reference is pulled in)."""
    import importlib
    import os
    import types

    root = os.environ.get("QUARTET_REF")
    qdir = os.path.join(root, "models", "quantization", "quantizers") if root else None
    if not qdir or not os.path.isfile(os.path.join(qdir, stem + ".py")):
        raise NotImplementedError(
            "this registry name is a plain-torch research baseline of the reference, outside the MXFP4 path this library "
            "accelerates; set QUARTET_REF to the `src` directory of a reference checkout to use the reference's own class")
    if _REF_PACKAGE not in sys.modules:
        pkg = types.ModuleType(_REF_PACKAGE)
        pkg.__path__ = [qdir]
        sys.modules[_REF_PACKAGE] = pkg
    return importlib.import_module(f"{_REF_PACKAGE}.{stem}")


def _reference_class(name: str, stem: str):
    def ctor(*a, **k):
        return getattr(_reference_module(stem), name)(*a, **k)

    ctor.__name__ = name
    return ctor


QUANTIZER_CLASSES = {name: _reference_class(name, stem) for stem, names in _OTHER_NAMES.items() for name in names.split()}
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
        self._handle = torch_ops.register_layer(self)  # names this layer to the quartet_b200::linear_* operators

    def __setstate__(self, state):
        super().__setstate__(state)
        self._handle = torch_ops.register_layer(self)  # a copy (deepcopy, unpickling) is a layer of its own

    def _fusable(self, x) -> bool:
        g = self.backward_scheme.g_quantizer
        aq, wq = self.activation_quantizer, self.weight_quantizer
        return (
            type(wq) is QuestMXFP4Quantizer
            and type(aq) is QuestMXFP4Quantizer
            and isinstance(g, AbsmaxRotation32)
            and type(self.backward_scheme) is QEQWtt_QEtQXtt_Scheme
            and g.rerotate in (None, "signs")
            and g._dense is None and aq._dense is None and wq._dense is None
            and aq._signs_dev is None and wq._signs_dev is None and aq._signs_host == 0 and wq._signs_host == 0
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
        if not wq.is_builtin_rotation or wq._sign_word() != 0:
            raise RuntimeError("only the plain 32-point Hadamard rotation is exported")
        with torch.no_grad():
            codes, sf, _ = ops.quant_fwd(self.weight.detach().contiguous(), wq.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=False)
        return codes, sf, wq.had_scale

    def forward(self, x):
        if self._fusable(x):
            if torch.is_autocast_enabled():
                out_dtype = torch.get_autocast_dtype("cuda")
                if out_dtype != torch.bfloat16:
                    out_dtype = torch.float32
            else:
                out_dtype = x.dtype
            sink = getattr(self, "wgrad_sink", None)
            if sink is None and torch.compiler.is_compiling():
                # one operator per direction: what torch.compile traces (and differentiates) without a graph break
                return torch_ops.quantized_linear(x, self.weight, self._handle, out_dtype)
            # eager: the same kernel sequence as a plain autograd function (less dispatch overhead per call)
            aq, wq = self.activation_quantizer, self.weight_quantizer
            aq._see(x)
            wq._see(self.weight)
            return QuartetLinearFn.apply(x, self.weight, aq, wq, self.backward_scheme.g_quantizer, out_dtype, sink)
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
