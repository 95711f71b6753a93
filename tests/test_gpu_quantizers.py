"""Parity of the CUDA quantizers (through the C ABI) with the CPU oracle and the golden vectors.

Bar: codes, scale bytes and mask bits are bit-exact.  The only admitted exceptions are counted and
must be explained by the oracle value sitting within 2 fp32 ulp of a rounding threshold (the
rotation is summed in a different order than the reference's 32-term dot) -- and on these inputs
the count is zero.
"""
import os

import numpy as np
import pytest
import torch

from oracle import ref_math as rm
from tests import helpers as H

pytestmark = pytest.mark.gpu

CASES = ["gauss", "grad", "student", "edge"]


@pytest.fixture(scope="module")
def ops():
    import __graft_entry__ as entry

    entry.build()
    from quartet_b200 import ops

    assert torch.cuda.is_available()
    return ops


@pytest.fixture(scope="module")
def gk(golden_dir):
    return np.load(os.path.join(golden_dir, "quantizer_kernel.npz"))


def _dev(x, dtype=torch.bfloat16):
    return x.to(dtype).cuda().contiguous()


def _check_fwd(ops, x, dtype, had_scale, h):
    rows, cols = x.shape
    ref = rm.quant_fwd(x, h)
    codes, sf, mask = ops.quant_fwd(_dev(x, dtype), had_scale=had_scale)
    torch.cuda.synchronize()
    idx, neg = H.unpack_codes(codes)
    e8 = H.unpack_sf(sf, rows, cols)
    n_sf, n_code, bad = H.compare_quantized(idx, neg, e8, ref)
    mask_bad = (H.unpack_mask(mask) != ref.mask) & ~(e8 != ref.e8m0).repeat_interleave(32, dim=1)
    # every code mismatch must be a boundary case
    v = (rm.rotate(x, h) / ref.shared.reshape(-1, 1)).abs().reshape(rows, cols)
    assert bool(H.near_threshold(v[bad], H.RTN_THRESHOLDS).all()), "code mismatch away from a rounding boundary"
    assert bool(H.near_threshold(v[mask_bad], torch.tensor([6.0])).all())
    return n_sf, n_code, int(mask_bad.sum())


@pytest.mark.parametrize("name", CASES)
def test_quant_fwd_golden_inputs(ops, gk, name):
    x = torch.from_numpy(gk[name + "_x"])
    n_sf, n_code, n_mask = _check_fwd(ops, x, torch.bfloat16, ops.HAD_SCALE_BF16, rm.hadamard32())
    assert (n_sf, n_code, n_mask) == (0, 0, 0)
    # and the de-quantized tensor equals what the reference kernel stored
    codes, sf, _ = ops.quant_fwd(_dev(x))
    out = ops.dequant(codes, sf, 1.0, torch.float32).cpu()
    ref = torch.from_numpy(gk[name + "_quest_out"])
    assert bool((out == ref).all())  # -0 == +0


@pytest.mark.parametrize("shape", [(1024, 1024), (200, 640), (128, 128), (1, 128)])
def test_quant_fwd_seeded(ops, shape):
    gen = torch.Generator().manual_seed(shape[0] * 7 + shape[1])
    x = H.bf16r(torch.randn(*shape, generator=gen))
    n_sf, n_code, n_mask = _check_fwd(ops, x, torch.bfloat16, ops.HAD_SCALE_BF16, rm.hadamard32())
    print(f"boundary exceptions {shape}: scale groups {n_sf}, codes {n_code}, mask bits {n_mask}")
    assert n_sf <= 1 and n_code <= 2 and n_mask <= 1


def test_quant_fwd_fp32_input(ops):
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(256, 512, generator=gen)
    n_sf, n_code, n_mask = _check_fwd(ops, x, torch.float32, ops.HAD_SCALE_F32, rm.hadamard32(torch.float32))
    assert n_sf <= 1 and n_code <= 2 and n_mask <= 1


def _bwd_ref_cmp(ops, codes, sf, ref, scale_tol_groups=0):
    idx, neg = H.unpack_codes(codes)
    e8 = H.unpack_sf(sf, ref.rows, ref.cols)
    n_sf, n_code, _ = H.compare_quantized(idx, neg, e8, ref)
    return n_sf, n_code


@pytest.mark.parametrize("name", CASES)
def test_quant_bwd_reference_stream_bit_exact(ops, gk, name):
    """Rounding mode 3 reproduces tl.rand(seed, offset): equals the reference kernel's own output."""
    x = torch.from_numpy(gk[name + "_x"])
    signs, seed = int(gk["signs"]), int(gk[name + "_sr_seed"])
    codes, sf = ops.quant_bwd(_dev(x), signs=signs, rounding=ops.ROUND_SR_TLRAND, seed=seed)
    out = ops.dequant(codes, sf, ops.SR_OPERAND_SCALE, torch.float32).cpu()
    ref = torch.from_numpy(gk[name + "_sr_out"])
    assert bool((out == ref).all())
    # round-to-nearest variant of the same quantizer
    codes, sf = ops.quant_bwd(_dev(x), signs=signs, rounding=ops.ROUND_NEAREST)
    out = ops.dequant(codes, sf, ops.SR_OPERAND_SCALE, torch.float32).cpu()
    assert bool((out == torch.from_numpy(gk[name + "_absmax_rtn_out"])).all())


def test_quant_bwd_noise_tensor_bit_exact(ops):
    gen = torch.Generator().manual_seed(11)
    x = H.bf16r(torch.randn(384, 512, generator=gen) * 1e-3)
    u = torch.rand(384, 512, generator=gen)
    signs = 0x9E3779B9
    h = rm.hadamard32()
    ref = rm.quant_bwd(x, h * rm.signs_to_diag(signs)[None, :], u)
    sd = torch.tensor([signs], dtype=torch.int64).cuda()
    codes, sf = ops.quant_bwd(_dev(x), signs_dev=sd, rounding=ops.ROUND_SR_NOISE, noise=u.cuda())
    assert _bwd_ref_cmp(ops, codes, sf, ref) == (0, 0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quant_bwd_own_stream(ops, dtype):
    gen = torch.Generator().manual_seed(3)
    x = H.bf16r(torch.randn(512, 1024, generator=gen) * 1e-3)
    h = rm.hadamard32()
    signs = 0x0F0F1234
    ref = rm.quant_bwd_own(x, h, signs, seed=0xDEADBEEF1234, offset=77)
    codes, sf = ops.quant_bwd(_dev(x, dtype), signs=signs, rounding=ops.ROUND_SR_PHILOX, seed=0xDEADBEEF1234, offset=77)
    n_sf, n_code = _bwd_ref_cmp(ops, codes, sf, ref)
    print("own-stream mismatches vs oracle:", n_sf, n_code)
    assert n_sf == 0 and n_code <= 4  # a last-ulp difference of the rotation can flip a dither decision
    # unbiased: |sum(q - v)| / sum|v| well inside 1e-3 (north-star bound)
    val = ops.dequant(codes, sf, ops.SR_OPERAND_SCALE, torch.float32).cpu()
    xh = rm.rotate(x, h * rm.signs_to_diag(signs)[None, :]).reshape(x.shape)
    rel = abs((val - xh).sum().item()) / xh.abs().sum().item()
    mag = ((val.abs() - xh.abs()).sum().item()) / xh.abs().sum().item()
    print("relative mean error:", rel, "magnitude bias:", mag)
    assert rel < 1e-3 and abs(mag) < 1e-3  # sampling noise at this size is ~3e-4; the large-sample test below is tighter
    # a different offset gives a different draw
    codes2, _ = ops.quant_bwd(_dev(x, dtype), signs=signs, rounding=ops.ROUND_SR_PHILOX, seed=0xDEADBEEF1234, offset=78)
    assert not bool((codes2 == codes).all())


def test_quant_bwd_own_stream_mean_over_draws(ops):
    """Averaging R independent draws converges to the rotated input like 1/sqrt(R)."""
    gen = torch.Generator().manual_seed(4)
    x = H.bf16r(torch.randn(128, 256, generator=gen))
    xd = _dev(x)
    xh = rm.rotate(x, rm.hadamard32()).reshape(x.shape)
    acc = torch.zeros_like(xh)
    R = 64
    for r in range(R):
        codes, sf = ops.quant_bwd(xd, rounding=ops.ROUND_SR_PHILOX, seed=99, offset=r)
        acc += ops.dequant(codes, sf, ops.SR_OPERAND_SCALE, torch.float32).cpu()
    err1 = ((ops.dequant(codes, sf, ops.SR_OPERAND_SCALE, torch.float32).cpu() - xh).norm() / xh.norm()).item()
    errR = ((acc / R - xh).norm() / xh.norm()).item()
    print("single draw", err1, "mean of", R, errR)
    assert errR < 1.5 * err1 / R ** 0.5


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (512, 128)])
def test_quant_bwd_t(ops, shape):
    gen = torch.Generator().manual_seed(shape[0] + shape[1])
    x = H.bf16r(torch.randn(*shape, generator=gen) * 1e-3)
    xt = x.T.contiguous()
    u = torch.rand(*xt.shape, generator=gen)
    h = rm.hadamard32()
    signs = 0x13572468
    ref = rm.quant_bwd(xt, h * rm.signs_to_diag(signs)[None, :], u)
    codes_t, sf_t = ops.quant_bwd_t(_dev(x), signs=signs, rounding=ops.ROUND_SR_NOISE, noise=u.cuda())
    assert _bwd_ref_cmp(ops, codes_t, sf_t, ref) == (0, 0)
    # reference-compatible stream over the transposed tensor
    ref3 = rm.quant_bwd(xt, h * rm.signs_to_diag(signs)[None, :], rm.triton_rand(4242, np.arange(xt.numel())).reshape(xt.shape))
    codes_t, sf_t = ops.quant_bwd_t(_dev(x), signs=signs, rounding=ops.ROUND_SR_TLRAND, seed=4242)
    assert _bwd_ref_cmp(ops, codes_t, sf_t, ref3) == (0, 0)
    # own stream, bf16 and fp32 sources
    refo = rm.quant_bwd_own(xt, h, signs, seed=5, offset=9)
    for dt in (torch.bfloat16, torch.float32):
        codes_t, sf_t = ops.quant_bwd_t(_dev(x, dt), signs=signs, rounding=ops.ROUND_SR_PHILOX, seed=5, offset=9)
        n_sf, n_code = _bwd_ref_cmp(ops, codes_t, sf_t, refo)
        assert n_sf == 0 and n_code <= 2


@pytest.mark.parametrize("shape", [(128, 128), (384, 256)])
def test_requant_t(ops, shape):
    gen = torch.Generator().manual_seed(21 + shape[0])
    x = H.bf16r(torch.randn(*shape, generator=gen))
    h = rm.hadamard32()
    fq = rm.quant_fwd(x, h)
    codes = fq.packed().cuda()
    sf = rm.to_blocked(fq.e8m0).cuda()
    xt = fq.dequant().T.contiguous()
    u = torch.rand(*xt.shape, generator=gen)
    signs = 0xCAFEF00D
    ref = rm.quant_bwd(xt, h * rm.signs_to_diag(signs)[None, :], u)
    codes_t, sf_t = ops.requant_t(codes, sf, 1.0, signs=signs, rounding=ops.ROUND_SR_NOISE, noise=u.cuda())
    assert _bwd_ref_cmp(ops, codes_t, sf_t, ref) == (0, 0)
    refo = rm.quant_bwd_own(xt, h, signs, seed=8, offset=1)
    codes_t, sf_t = ops.requant_t(codes, sf, 1.0, signs=signs, rounding=ops.ROUND_SR_PHILOX, seed=8, offset=1)
    n_sf, n_code = _bwd_ref_cmp(ops, codes_t, sf_t, refo)
    assert n_sf == 0 and n_code <= 2


def test_dequant_and_unrotate(ops):
    gen = torch.Generator().manual_seed(31)
    packed, e8, val = H.random_mxfp4(200, 256, gen)
    out = ops.dequant(packed.cuda(), rm.to_blocked(e8).cuda(), 1.0, torch.float32).cpu()
    assert bool((out == val).all())
    outb = ops.dequant(packed.cuda(), rm.to_blocked(e8).cuda(), 4.0 / 3.0, torch.bfloat16).cpu().float()
    assert bool((outb == (val * torch.tensor(4.0 / 3.0)).to(torch.bfloat16).float()).all())
    g = torch.randn(200, 256, generator=gen)
    m = torch.rand(200, 256, generator=gen) < 0.9
    q = rm.Quantized(200, 256, None, None, None, None, m)
    ref = rm.unrotate_mask(g, m, rm.hadamard32())
    got = ops.unrotate_mask(g.cuda(), q.packed_mask().cuda(), ops.HAD_SCALE_BF16).cpu()
    assert (got - ref).norm() / ref.norm() < 1e-6
    got = ops.unrotate_mask(g.cuda().bfloat16(), None, ops.HAD_SCALE_BF16, out_dtype=torch.float32).cpu()
    ref = rm.unrotate_mask(H.bf16r(g), torch.ones_like(m), rm.hadamard32())
    assert (got - ref).norm() / ref.norm() < 1e-6


def test_roundtrip_property_large(ops):
    """Size-independent property at a bench-sized tensor: quantize -> dequantize -> quantize is
    idempotent for the forward quantizer's codes when fed its own rotated output un-rotated back,
    and the relative error of the forward quantizer sits in the expected band."""
    torch.manual_seed(0)
    x = torch.randn(16384, 4096, device="cuda", dtype=torch.bfloat16)
    codes, sf, mask = ops.quant_fwd(x)
    val = ops.dequant(codes, sf, 1.0, torch.float32)
    xr = ops.unrotate_mask(val, None, ops.HAD_SCALE_BF16)  # rotate back (H is symmetric, orthonormal up to bf16 rounding)
    rel = ((xr - x.float()).norm() / x.float().norm()).item()
    print("fwd quantizer relative error", rel)
    assert 0.08 < rel < 0.22
    # own-stream stochastic rounding at the same size: unbiased in value and in magnitude
    # (north-star bound 1e-3; 67 M elements put the sampling noise near 3e-5)
    e = x * 1e-3
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    h = rm.hadamard32().cuda()
    xh = (e.float().reshape(-1, 32) @ h).reshape(e.shape)
    torch.backends.cuda.matmul.allow_tf32 = prev
    codes, sf = ops.quant_bwd(e, rounding=ops.ROUND_SR_PHILOX, seed=12345, offset=1)
    val = ops.dequant(codes, sf, ops.SR_OPERAND_SCALE, torch.float32)
    denom = xh.abs().double().sum()
    signed = ((val - xh).double().sum() / denom).abs().item()
    mag = ((val.abs() - xh.abs()).double().sum() / denom).item()
    print("SR relative mean error", signed, "magnitude bias", mag)
    assert signed < 1e-4 and abs(mag) < 1e-4
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rounding", [0, 1])
def test_quant_bwd_dual_equals_the_two_separate_quantizers(ops, dtype, rounding):
    """One read of E: the row-wise half is quant_bwd bit for bit, the transposed half quant_bwd_t bit for bit
    (different seeds for the two, a non-trivial sign vector, a ragged number of tiles per SM)."""
    g = torch.Generator().manual_seed(404)
    x = (torch.randn(640, 384, generator=g) * 3e-3).to(dtype).cuda()
    kw = dict(signs=0x9E3779B9, rounding=rounding)
    c, s, ct, st = ops.quant_bwd_dual(x, ops.HAD_SCALE_BF16, seed_rows=11, seed_t=22, offset=5, **kw)
    c1, s1 = ops.quant_bwd(x, ops.HAD_SCALE_BF16, seed=11, offset=5, **kw)
    c2, s2 = ops.quant_bwd_t(x, ops.HAD_SCALE_BF16, seed=22, offset=5, **kw)
    assert torch.equal(c, c1) and torch.equal(s, s1)
    assert torch.equal(ct, c2) and torch.equal(st, s2)
    with pytest.raises(ValueError):
        ops.quant_bwd_dual(x[:100], ops.HAD_SCALE_BF16)  # rows not a multiple of 128
    assert ops.device_status() == 0


def test_a_wait_that_runs_out_sets_the_fault_word_and_leaves_the_context_usable(ops):
    """Every wait in the kernels is bounded; this drives one to its limit on purpose-built ground (a barrier nothing
    completes, 4096 polls): the kernel returns, the fault word names the wait, is cleared by reading it, and the next
    kernel runs normally."""
    from quartet_b200 import _lib

    assert ops.device_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _lib.load().quartet_selftest_wait_timeout(flag.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    word = ops.device_status()
    assert flag.item() == 1 and word & 0x100 and (word & 0xFF) == 1  # "gave up" bit + the code of a load wait
    assert ops.device_status() == 0                                    # reading cleared it
    x = torch.randn(128, 128, device="cuda", dtype=torch.bfloat16)
    codes, sf, mask = ops.quant_fwd(x)
    assert torch.isfinite(ops.dequant(codes, sf).sum()).item() and ops.device_status() == 0
