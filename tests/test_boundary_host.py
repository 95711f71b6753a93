"""Host-side checks of the reference-facing boundary that need no GPU: the operators' shape contracts
(their fake kernels, the ones the reference's notebook registers for the real-quantized operators it calls,
notebooks/benchmark_mxfp4.ipynb:881-958), tracing a whole layer through them, the registry, and -- when a
reference checkout is named by QUARTET_REF -- the reference's own model code resolving to this package."""
import os
import sys
import textwrap

import pytest
import torch

import quartet_b200.quantization as Q
import quartet_b200.torch_ops  # noqa: F401  (registers the operators)
from quartet_b200 import ops

T = torch.ops.quartet_b200


def _meta(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, dtype=dtype, device="meta")


def test_operator_shape_contracts():
    m, k, n = 384, 512, 256
    x, w = _meta(m, k), _meta(n, k)
    codes, sf, mask = T.quant_fwd(x, 0.1767578125, 0.487)
    # fusedQuantizeMx: e2m1 [M, K/2], e8m0 [pad128(M), pad4(K/32)] (blocked, flat here), mask [M, K/8]
    assert codes.shape == (m, k // 2) and sf.shape == (384 * 16,) and mask.shape == (m, k // 8)
    assert codes.dtype == sf.dtype == mask.dtype == torch.uint8
    e = _meta(m, n)
    ct, st = T.quant_bwd_t(e, 0.1767578125, 0, None, 1, 0, 0, None)       # backward_t_bf16: e2m1 [N, M/2], e8m0 [N, M/32]
    assert ct.shape == (n, m // 2) and st.shape == (ops.sf_bytes(n, m),)
    rc, rs = T.requant_t(codes, sf, 1.0, 0.1767578125, 0, None, 1, 0, 0, None)  # backward_qt_bf16: [K, M/2], [K, M/32]
    assert rc.shape == (k, m // 2) and rs.shape == (ops.sf_bytes(k, m),)
    d = T.quant_bwd_dual(e, 0.1767578125, 0, None, 1, 0, 0, 0)
    assert [t.shape for t in d] == [(m, n // 2), (ops.sf_bytes(m, n),), (n, m // 2), (ops.sf_bytes(n, m),)]
    wc, ws, _ = T.quant_fwd(w, 0.1767578125, 0.487)
    y = T.gemm_mxfp4_tn(codes, sf, wc, ws, 1.0, None, 0.1767578125, torch.bfloat16)   # matmul_mxf4_bf16_tn: bf16 [M, N]
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    assert T.dequant(codes, sf, 1.0, torch.float32).shape == (m, k)
    assert T.unrotate_mask(y, None, 0.1767578125, torch.float32).dtype == torch.float32
    with pytest.raises(RuntimeError):
        T.gemm_mxfp4_tn(codes, sf, _meta(n, 100, dtype=torch.uint8), ws, 1.0, None, 0.17, torch.bfloat16)  # K mismatch


def _production_linear(k, n):
    return Q.QuantizedLinear(
        k, n, bias=False,
        weight_quantizer=Q.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
        activation_quantizer=Q.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
        gradient_quantizer=Q.QUANTIZER_CLASSES["AlbertTsengQuantizer"](stochastic=True, rerotate="signs"),
        backward_scheme=Q.BACKWARD_SCHEMES["Q(E)Q(Wt)t_Q(Et)Q(Xt)t"](),
    )


def test_layer_traces_to_one_operator_per_direction():
    """Forward and backward of QuantizedLinear, traced symbolically (fake CUDA tensors, no device needed): the
    graph holds exactly one quartet_b200::linear_fwd and one quartet_b200::linear_bwd, with a ragged token count
    (padded to 128 inside) and the shapes autograd expects."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from torch.fx.experimental.proxy_tensor import make_fx

    lin = _production_linear(256, 384)
    handle = lin._handle

    def fwd_bwd(x, w, e):
        y = torch.ops.quartet_b200.linear_fwd(x, w, handle, torch.bfloat16)
        dx, dw = torch.ops.quartet_b200.linear_bwd(e, *y[1:], handle, x.dtype, w.dtype, True, True)
        return y[0], dx, dw

    with FakeTensorMode() as mode:
        x = torch.empty(3, 50, 256, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(384, 256, dtype=torch.float32, device="cuda")
        e = torch.empty(3, 50, 384, dtype=torch.bfloat16, device="cuda")
        gm = make_fx(fwd_bwd)(x, w, e)
        y, dx, dw = fwd_bwd(x, w, e)
    names = [str(n.target) for n in gm.graph.nodes if n.op == "call_function"]
    assert sum("linear_fwd" in t for t in names) == 1 and sum("linear_bwd" in t for t in names) == 1
    assert y.shape == (3, 50, 384) and y.dtype == torch.bfloat16
    assert dx.shape == (150, 256) and dx.dtype == torch.bfloat16 and dw.shape == (384, 256) and dw.dtype == torch.float32


def test_producer_fused_layer_operators_trace():
    """rmsnorm_linear_fwd / swiglu_linear_fwd (the layer with the step that produces its input inside the forward
    quantizer): shape contracts of their fake kernels, on fake CUDA tensors (their backward needs a device's
    autograd engine and is covered by the GPU tests)."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    ln = _production_linear(256, 384)
    proj = _production_linear(512, 256)
    with FakeTensorMode():
        x = torch.empty(3, 50, 256, dtype=torch.float32, device="cuda")
        gamma = torch.empty(256, dtype=torch.float32, device="cuda")
        w = torch.empty(384, 256, dtype=torch.float32, device="cuda")
        out = T.rmsnorm_linear_fwd(x, gamma, 1e-5, w, ln._handle, torch.bfloat16)
        assert out[0].shape == (3, 50, 384) and out[0].dtype == torch.bfloat16 and out[1].shape == (256, 128)
        assert out[7].shape == (3, 50, 1) and out[7].dtype == torch.float32
        h = torch.empty(3, 50, 1024, dtype=torch.bfloat16, device="cuda")
        w2 = torch.empty(256, 512, dtype=torch.float32, device="cuda")
        out = T.swiglu_linear_fwd(h, w2, proj._handle, torch.bfloat16)
        assert out[0].shape == (3, 50, 256) and out[1].shape == (256, 256) and out[3].shape == (256, 64)


def test_registry_names_and_module_attributes():
    assert len(Q.QUANTIZER_CLASSES) == 40
    assert set(Q.BACKWARD_SCHEMES) == {"EW_EtX", "Q(E)W_Q(Et)X", "Q(E)Q(Wt)t_Q(Et)Q(Xt)t"}
    q = Q.QUANTIZER_CLASSES["AlbertTsengQuantizer"](hadamard_dim=32, stochastic=True, rerotate="signs")
    assert (q.bits, q.n_levels, q.hadamard_dim, q.rerotate, q.stochastic) == (4, 16, 32, "signs", True)
    hm = q.hadamard_matrix
    assert hm.shape == (32, 32) and torch.allclose(hm @ hm.T, torch.eye(32), atol=1e-6)
    q.hadamard_matrix = -hm  # assigning a sign-flipped Sylvester matrix keeps the built-in rotation
    assert q.is_builtin_rotation and q._sign_word() == 0xFFFFFFFF
    q.hadamard_matrix = torch.linalg.qr(torch.randn(32, 32, generator=torch.Generator().manual_seed(0)))[0]
    assert not q.is_builtin_rotation  # a general matrix is kept as it is
    q64 = Q.QUANTIZER_CLASSES["AlignedAlbertTsengQuantizer"](hadamard_dim=64)
    assert q64.hadamard_matrix.shape == (64, 64) and not q64.is_builtin_rotation and q64.stochastic is False
    with pytest.raises(ValueError):
        Q.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](hadamard_dim=48)
    with pytest.raises(ValueError):
        Q.QUANTIZER_CLASSES["AlbertTsengQuantizer"](rerotate="bogus")
    lin = _production_linear(128, 128)
    assert list(lin.state_dict().keys()) == ["weight"]  # quantizers add no checkpoint keys
    assert lin.backward_scheme.g_quantizer.rerotate == "signs"


def test_other_registry_names_build_the_reference_class_from_a_checkout(tmp_path, monkeypatch):
    """A name outside the MXFP4 path is served by the class a reference checkout defines (a stand-in tree here)."""
    qdir = tmp_path / "models" / "quantization" / "quantizers"
    qdir.mkdir(parents=True)
    (qdir / "base.py").write_text("import torch.nn as nn\nclass BaseQuantizer(nn.Module):\n    def __init__(self, bits=4):\n        super().__init__()\n        self.bits = bits\n")
    (qdir / "noise.py").write_text(textwrap.dedent("""
        from .base import BaseQuantizer
        class NoiseQuantizer(BaseQuantizer):
            def __init__(self, bits=4, marker="from the checkout"):
                super().__init__(bits)
                self.marker = marker
            def forward(self, x):
                return x
    """))
    monkeypatch.delenv("QUARTET_REF", raising=False)
    monkeypatch.delitem(sys.modules, "quartet_reference_quantizers", raising=False)
    monkeypatch.delitem(sys.modules, "quartet_reference_quantizers.noise", raising=False)
    with pytest.raises(NotImplementedError):
        Q.QUANTIZER_CLASSES["NoiseQuantizer"]()
    monkeypatch.setenv("QUARTET_REF", str(tmp_path))
    q = Q.QUANTIZER_CLASSES["NoiseQuantizer"](bits=8)
    assert q.marker == "from the checkout" and q.bits == 8
    with pytest.raises(NotImplementedError):  # a file the stand-in tree does not have
        Q.QUANTIZER_CLASSES["PACTQuantizer"]()
    for name in ("quartet_reference_quantizers", "quartet_reference_quantizers.noise", "quartet_reference_quantizers.base"):
        sys.modules.pop(name, None)


@pytest.mark.skipif(__import__("tests.ref_model", fromlist=["x"]).reference_src() is None,
                    reason="needs a reference checkout: set QUARTET_REF to its `src` directory")
def test_reference_model_code_resolves_to_this_package():
    """The reference's own `models/llama.py`, unchanged, builds its 30M configuration on top of this package once
    `install()` has registered it as `models.quantization` (src/models/llama.py:14, 89-110), with the reference's own
    argument parser and the flags of its launch script."""
    from tests.ref_model import reference_on_this_package

    with reference_on_this_package() as (llama, args):
        assert args.w_quant == "QuestMXFP4Quantizer" and args.g_quant_kwargs == {"stochastic": True, "rerotate": "signs"}
        model = llama.Llama(args)
        linears = [m for m in model.modules() if isinstance(m, Q.QuantizedLinear)]
        assert len(linears) == 24  # four per block, six blocks
        shapes = sorted({(m.out_features, m.in_features) for m in linears})
        assert shapes == [(640, 640), (640, 1792), (1920, 640), (3584, 640)]  # SwiGLU hidden size 1792 (multiple_of 256)
        for m in linears:
            assert type(m.weight_quantizer) is Q.QuestMXFP4Quantizer and type(m.activation_quantizer) is Q.QuestMXFP4Quantizer
            g = m.backward_scheme.g_quantizer
            assert type(g) is Q.AlbertTsengQuantizer and g.stochastic and g.rerotate == "signs"
            assert type(m.backward_scheme).__name__ == "QEQWtt_QEtQXtt_Scheme" and m.bias is None
        assert not isinstance(model.lm_head, Q.QuantizedLinear)
        assert sum(p.numel() for p in model.parameters()) > 70_000_000  # 30.5 M in the blocks, untied 32000 x 640 embeddings twice


def test_producer_calls_fall_back_to_the_separate_steps():
    """Where the fused form does not apply (here: CPU tensors, un-quantized layers), rmsnorm_linear / swiglu_linear are
    the norm / activation followed by the layer, gradients included."""
    torch.manual_seed(0)
    lin = Q.QuantizedLinear(64, 48, bias=False)
    x = torch.randn(3, 7, 64, requires_grad=True)
    gamma = (1.0 + 0.1 * torch.randn(64)).requires_grad_(True)
    y = Q.rmsnorm_linear(x, gamma, 1e-5, lin)
    want = lin((x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)) * gamma)
    assert torch.allclose(y, want, atol=1e-6)
    y.sum().backward()
    assert x.grad is not None and gamma.grad is not None and lin.weight.grad is not None
    proj = Q.QuantizedLinear(32, 16, bias=False)
    h = torch.randn(5, 64, requires_grad=True)
    z = Q.swiglu_linear(h, proj)
    assert torch.allclose(z, proj(torch.nn.functional.silu(h[:, :32]) * h[:, 32:]), atol=1e-6)
    z.sum().backward()
    assert h.grad is not None and h.grad.shape == h.shape
