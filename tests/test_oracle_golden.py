"""The CPU oracle against the golden vectors produced by the reference's own code
(tests/golden/make_golden.py).  Bit-exact, no tolerance."""
import os

import numpy as np
import pytest
import torch

from oracle import ref_math as rm

CASES = ["gauss", "grad", "student", "edge"]


def _same(a, b):
    return bool(((a == b) | (torch.isnan(a) & torch.isnan(b))).all())


@pytest.fixture(scope="module")
def gk(golden_dir):
    return np.load(os.path.join(golden_dir, "quantizer_kernel.npz"))


@pytest.mark.parametrize("name", CASES)
def test_quest_branch_bit_exact(gk, name):
    h = rm.hadamard32()
    q = rm.quant_fwd(torch.from_numpy(gk[name + "_x"]), h)
    assert _same(q.dequant(), torch.from_numpy(gk[name + "_quest_out"]))
    assert bool((q.mask == torch.from_numpy(gk[name + "_quest_mask"])).all())
    # the derived bytes mean the same values the reference stored
    assert _same(q.dequant_from_bytes(), q.dequant())


@pytest.mark.parametrize("name", CASES)
def test_sr_branch_bit_exact_with_triton_philox(gk, name):
    h = rm.hadamard32()
    hb = h * rm.signs_to_diag(int(gk["signs"]))[None, :]
    x = torch.from_numpy(gk[name + "_x"])
    u = rm.triton_rand(int(gk[name + "_sr_seed"]), np.arange(x.numel())).reshape(x.shape)
    q = rm.quant_bwd(x, hb, u)
    assert _same(q.dequant(), torch.from_numpy(gk[name + "_sr_out"]))
    if name != "edge":  # all-zero groups dequantise to -0 * 0 in the reference; bytes say the same
        assert _same(q.dequant_from_bytes(), q.dequant())


@pytest.mark.parametrize("name", CASES)
def test_absmax_rtn_branch_bit_exact(gk, name):
    h = rm.hadamard32()
    hb = h * rm.signs_to_diag(int(gk["signs"]))[None, :]
    q = rm.quant_bwd(torch.from_numpy(gk[name + "_x"]), hb, None, stochastic=False)
    assert _same(q.dequant(), torch.from_numpy(gk[name + "_absmax_rtn_out"]))


def test_sign_vector_is_a_sign_bit_flip(gk):
    """Rotating with H @ diag(s) only flips code sign bits, so the kernels apply `signs` that way."""
    h = rm.hadamard32()
    signs = int(gk["signs"])
    x = torch.from_numpy(gk["gauss_x"])
    u = rm.triton_rand(7, np.arange(x.numel())).reshape(x.shape)
    a = rm.quant_bwd(x, h * rm.signs_to_diag(signs)[None, :], u)
    b = rm.quant_bwd(x, h, u)
    flip = torch.tensor([bool((signs >> j) & 1) for j in range(32)]).repeat(x.shape[1] // 32)
    assert bool((a.idx == b.idx).all()) and bool((a.neg == (b.neg ^ flip)).all())
    assert bool((a.e8m0 == b.e8m0).all())


def test_layer_forward_backward_bit_exact(golden_dir):
    g = np.load(os.path.join(golden_dir, "linear_fwd_bwd.npz"))
    h = rm.hadamard32()
    x, w, e = (torch.from_numpy(g[k]) for k in "xwe")
    hb = h * rm.signs_to_diag(int(g["signs"]))[None, :]
    y, xq, wq = rm.linear_forward(x, w, h)
    assert _same(y, torch.from_numpy(g["y"]))
    dx, dw, _, _ = rm.linear_backward(e, xq, wq, h, hb, seeds=[int(s) for s in g["seeds"]])
    assert _same(dx, torch.from_numpy(g["dx"]))
    assert _same(dw, torch.from_numpy(g["dw"]))


def test_notebook_error_bands():
    """Squared relative L2 bands asserted in notebooks/benchmark_mxfp4.ipynb:620-634."""
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(128, 4096, generator=gen).bfloat16().float()
    w = torch.randn(128, 4096, generator=gen).bfloat16().float()
    h = rm.hadamard32()
    y_ref = x @ w.T
    y, xq, wq = rm.linear_forward(x, w, h)
    err = ((y - y_ref).norm() / y_ref.norm()).pow(2).item()
    assert 2e-2 < err < 6e-2
    e = torch.randn(128, 128, generator=gen).bfloat16().float()
    noises = [torch.rand(s, generator=gen) for s in ((128, 128), (4096, 128), (128, 128), (4096, 128))]
    dx, dw, _, _ = rm.linear_backward(e, xq, wq, h, h, noises=noises)
    gw_ref = e.T @ x
    gerr = ((dw - gw_ref).norm() / gw_ref.norm()).pow(2).item()
    assert 6e-2 < gerr < 15e-2


def test_blocked_layout_roundtrip():
    e = torch.randint(0, 255, (200, 10), dtype=torch.uint8)
    b = rm.to_blocked(e)
    assert b.numel() == 256 * 12
    assert bool((rm.from_blocked(b, 200, 10) == e).all())
    for r, c in ((0, 0), (31, 3), (32, 0), (127, 3), (128, 4), (199, 9)):
        assert int(b[rm.sf_offset(r, c, 12)]) == int(e[r, c])


def test_own_stream_is_unbiased():
    """Own dither stream: aggregate |sum(q - v)| / sum|v| far below 1e-3, and bit-stable."""
    gen = torch.Generator().manual_seed(1)
    x = (torch.randn(512, 1024, generator=gen) * 1e-3).bfloat16().float()
    h = rm.hadamard32()
    q = rm.quant_bwd_own(x, h, 0, seed=123, offset=0)
    xh = rm.rotate(x, h).reshape(x.shape)
    d = q.dequant_from_bytes()
    rel = abs((d - xh).sum().item()) / xh.abs().sum().item()
    assert rel < 1e-3
    q2 = rm.quant_bwd_own(x, h, 0, seed=123, offset=0)
    assert bool((q.codes == q2.codes).all())
    assert int(q.idx.max()) <= 7 and int(q.idx.min()) >= 0


@pytest.mark.parametrize("name", ["f32", "bf16"])
def test_producer_steps_equal_the_reference_models_own(golden_dir, name):
    """oracle.ref_math.rmsnorm / swiglu against the reference's `RMSNorm` module and `LlamaMLP.forward`
    (src/models/llama.py:64-75, 112-114; fixture tests/golden/producer_steps.npz, generator
    tests/golden/make_producer_golden.py): bit for bit, fp32 and bf16 inputs."""
    g = np.load(os.path.join(golden_dir, "producer_steps.npz"))

    def tensor(key):
        a = torch.from_numpy(g[key])
        return a.view(torch.bfloat16) if a.dtype == torch.int16 else a

    x, want = tensor(f"rms_x_{name}"), tensor(f"rms_out_{name}")
    got = rm.rmsnorm(x, torch.from_numpy(g["rms_weight"]), float(g["rms_eps"]))
    assert got.dtype == torch.float32 and torch.equal(got, want)
    # with the row statistic handed in (what the device tests do), the remaining steps give the same bits
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + float(g["rms_eps"]))
    assert torch.equal(rm.rmsnorm(x, torch.from_numpy(g["rms_weight"]), float(g["rms_eps"]), rstd=rstd), want)
    h, want = tensor(f"swiglu_h_{name}"), tensor(f"swiglu_out_{name}")
    got = rm.swiglu(h)
    assert got.dtype == h.dtype and torch.equal(got.float(), want.float())
