"""Parity at the shapes the headline configurations are quoted on (all through the C ABI):

* config 1: X [8192, 640], W [2560, 640], E [8192, 2560]; every quantizer and the three GEMMs against the
  oracle's whole-layer forward / backward;
* config 3: bf16 [4096, K], K in {4096, 8192, 14336}, Student-t(3) with 1 % of the channels x20;
* config 4: one GEMM per distinct extent (K = 11008, N = 22016, contraction over 16384 tokens);
* the two-CTA GEMM with a ragged last column tile (N = 1920, the 30M model's fused QKV projection);
* constructed inputs whose rotated, scaled values sit EXACTLY on a rounding tie.

Bar: codes, scale bytes and mask bits bit-exact; every admitted exception is counted and must lie within
2 fp32 ulp of a rounding threshold (the 32-term rotation is summed as a butterfly here, as a dot product in
the reference).  GEMMs: <= 1e-5 relative Frobenius error with fp32 output (bound of the path: 1e-2).
"""
import numpy as np
import pytest
import torch

from oracle import ref_math as rm
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import __graft_entry__ as entry

    entry.build()
    from quartet_b200 import ops

    return ops


def _fwd_exceptions(ops, x, dtype=torch.bfloat16, had_scale=None, h=None):
    """(scale groups, codes, mask bits) that differ from the oracle; asserts each is a boundary case."""
    h = rm.hadamard32() if h is None else h
    had_scale = ops.HAD_SCALE_BF16 if had_scale is None else had_scale
    rows, cols = x.shape
    ref = rm.quant_fwd(x, h)
    codes, sf, mask = ops.quant_fwd(x.to(dtype).cuda().contiguous(), had_scale=had_scale)
    idx, neg = H.unpack_codes(codes)
    e8 = H.unpack_sf(sf, rows, cols)
    n_sf, n_code, bad = H.compare_quantized(idx, neg, e8, ref)
    mask_bad = (H.unpack_mask(mask) != ref.mask) & ~(e8 != ref.e8m0).repeat_interleave(32, dim=1)
    v = (rm.rotate(x, h) / ref.shared.reshape(-1, 1)).abs().reshape(rows, cols)
    assert bool(H.near_threshold(v[bad], H.RTN_THRESHOLDS).all()), "code mismatch away from a rounding boundary"
    assert bool(H.near_threshold(v[mask_bad], torch.tensor([6.0])).all()), "mask mismatch away from the clip boundary"
    return n_sf, n_code, int(mask_bad.sum()), (codes, sf, mask), ref


def _bwd_cmp(codes, sf, ref):
    idx, neg = H.unpack_codes(codes)
    e8 = H.unpack_sf(sf, ref.rows, ref.cols)
    n_sf, n_code, _ = H.compare_quantized(idx, neg, e8, ref)
    return n_sf, n_code


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


# ------------------------------------------------------------------------------------------------
# config 1: the whole layer
# ------------------------------------------------------------------------------------------------
def test_config1_layer_every_quantizer_and_gemm(ops):
    gen = torch.Generator().manual_seed(0)
    x = H.bf16r(torch.randn(8192, 640, generator=gen))
    w = H.bf16r(torch.randn(2560, 640, generator=gen) * 0.02)
    e = H.bf16r(torch.randn(8192, 2560, generator=gen) * 1e-3)
    s = torch.randint(0, 2, (32,), generator=gen) * 2 - 1
    signs = sum(1 << j for j in range(32) if s[j] < 0)
    h_f = rm.hadamard32()
    h_b = h_f * rm.signs_to_diag(signs)[None, :]

    # forward quantizers (Q1) and forward GEMM (G1)
    nx = _fwd_exceptions(ops, x)
    nw = _fwd_exceptions(ops, w)
    print("config 1 forward exceptions (scale groups, codes, mask bits): X", nx[:3], "W", nw[:3])
    assert nx[:3] == (0, 0, 0) and nw[:3] == (0, 0, 0)
    (xc, xs, xm), xq = nx[3], nx[4]
    (wc, ws, wm), wq = nw[3], nw[4]
    y = ops.gemm_mxfp4_tn(xc, xs, wc, ws, 1.0, out_dtype=torch.float32).cpu()
    y_ref = xq.dequant() @ wq.dequant().T
    assert _rel(y, y_ref) < 1e-5

    # backward quantizers with the noise tensors the oracle uses, in the reference's call order
    # E, Wq^T, E^T, Xq^T (backward.py:69-83)
    shapes = [(8192, 2560), (640, 2560), (2560, 8192), (640, 8192)]
    noises = [torch.rand(sh, generator=gen) for sh in shapes]
    dx_ref, dw_ref, (eq, wtq, etq, xtq), _ = rm.linear_backward(e, xq, wq, h_f, h_b, noises=noises)
    R = ops.ROUND_SR_NOISE
    ed = e.bfloat16().cuda()
    ec, es = ops.quant_bwd(ed, signs=signs, rounding=R, noise=noises[0].cuda())                 # Q2
    wtc, wts = ops.requant_t(wc, ws, 1.0, signs=signs, rounding=R, noise=noises[1].cuda())      # Q4 on Wq
    etc_, ets = ops.quant_bwd_t(ed, signs=signs, rounding=R, noise=noises[2].cuda())            # Q3
    xtc, xts = ops.requant_t(xc, xs, 1.0, signs=signs, rounding=R, noise=noises[3].cuda())      # Q4 on Xq
    for name, got, ref in (("Q(E)", (ec, es), eq), ("Q(Wq^T)", (wtc, wts), wtq), ("Q(E^T)", (etc_, ets), etq),
                           ("Q(Xq^T)", (xtc, xts), xtq)):
        n_sf, n_code = _bwd_cmp(*got, ref)
        print("config 1", name, "scale groups", n_sf, "codes", n_code)
        assert n_sf == 0 and n_code <= 2, name
    a = ops.SR_OPERAND_SCALE ** 2
    dx = ops.gemm_mxfp4_tn(ec, es, wtc, wts, a, mask=xm, out_dtype=torch.float32).cpu()         # G2 + U1
    dw = ops.gemm_mxfp4_tn(etc_, ets, xtc, xts, a, mask=wm, out_dtype=torch.float32).cpu()      # G3 + U1
    print("config 1 rel err: y", _rel(y, y_ref), "dx", _rel(dx, dx_ref), "dw", _rel(dw, dw_ref))
    assert _rel(dx, dx_ref) < 1e-5 and _rel(dw, dw_ref) < 1e-5
    # bf16 results (what the autograd function returns under autocast) stay inside the path's bound
    dxb = ops.gemm_mxfp4_tn(ec, es, wtc, wts, a, mask=xm, out_dtype=torch.bfloat16).cpu().float()
    assert _rel(dxb, dx_ref) < 1e-2
    # the dual-output quantizer on the same E equals the two single-output ones
    c, s_, ct, st = ops.quant_bwd_dual(ed, signs=signs, rounding=ops.ROUND_SR_PHILOX, seed_rows=3, seed_t=4)
    c1, s1 = ops.quant_bwd(ed, signs=signs, rounding=ops.ROUND_SR_PHILOX, seed=3)
    c2, s2 = ops.quant_bwd_t(ed, signs=signs, rounding=ops.ROUND_SR_PHILOX, seed=4)
    assert torch.equal(c, c1) and torch.equal(s_, s1) and torch.equal(ct, c2) and torch.equal(st, s2)
    assert ops.device_status() == 0


# ------------------------------------------------------------------------------------------------
# config 3: the quantize-only sweep's distribution, at its parity size M = 4096
# ------------------------------------------------------------------------------------------------
def student_t_with_outliers(m, k, seed=0):
    rng = np.random.default_rng(seed)
    x = rng.standard_t(3, (m, k)).astype(np.float32)
    ch = rng.choice(k, round(0.01 * k), replace=False)
    x[:, ch] *= 20
    return H.bf16r(torch.from_numpy(x))


@pytest.mark.parametrize("k", [4096, 8192, 14336])
def test_config3_quantizers_bit_exact(ops, k):
    m = 4096
    x = student_t_with_outliers(m, k)
    n_sf, n_code, n_mask, _, _ = _fwd_exceptions(ops, x)
    print(f"config 3 K={k} forward exceptions: scale groups {n_sf}, codes {n_code}, mask bits {n_mask} of {m * k} elements")
    assert n_sf == 0 and n_code <= 4 and n_mask <= 2
    gen = torch.Generator().manual_seed(k)
    signs = 0x5A5AC3C3
    h_b = rm.hadamard32() * rm.signs_to_diag(signs)[None, :]
    xd = x.bfloat16().cuda()
    u = torch.rand(m, k, generator=gen)
    ref = rm.quant_bwd(x, h_b, u)
    # the butterfly rotation differs from the reference's dot product in the last ulp of some values, which can
    # flip a stochastic decision only when |u - p| < ~1e-7: well under one expected flip per 10^7 elements
    n_sf, n_code = _bwd_cmp(*ops.quant_bwd(xd, signs=signs, rounding=ops.ROUND_SR_NOISE, noise=u.cuda()), ref)
    print(f"config 3 K={k} row-wise backward quantizer: scale groups {n_sf}, codes {n_code}")
    assert n_sf == 0 and n_code <= 3
    del ref
    xt = x.T.contiguous()
    ut = torch.rand(k, m, generator=gen)
    ref_t = rm.quant_bwd(xt, h_b, ut)
    n_sf, n_code = _bwd_cmp(*ops.quant_bwd_t(xd, signs=signs, rounding=ops.ROUND_SR_NOISE, noise=ut.cuda()), ref_t)
    print(f"config 3 K={k} transposing backward quantizer: scale groups {n_sf}, codes {n_code}")
    assert n_sf == 0 and n_code <= 3
    assert ops.device_status() == 0


# ------------------------------------------------------------------------------------------------
# config 4: one GEMM per distinct extent of the 7B layers
# ------------------------------------------------------------------------------------------------
def _random_operand_dev(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    codes = torch.randint(0, 256, (rows, cols // 2), generator=g, device="cuda", dtype=torch.uint8)
    e8 = torch.randint(118, 130, (rows, cols // 32), generator=g, device="cuda", dtype=torch.uint8)
    return codes, e8


def _values(codes_u8, e8):
    """CPU float64 values of packed codes + logical scale bytes."""
    c = codes_u8.cpu()
    full = torch.stack([c & 0xF, c >> 4], dim=-1).reshape(c.shape[0], -1)
    grid = torch.tensor(rm.E2M1_GRID, dtype=torch.float64)
    val = grid[(full & 7).long()] * torch.where((full & 8) != 0, -1.0, 1.0)
    return (val.reshape(c.shape[0], -1, 32) * torch.exp2(e8.cpu().double() - 127).unsqueeze(-1)).reshape(c.shape[0], -1)


@pytest.mark.parametrize("mnk,fused,out", [((16384, 4096, 11008), False, torch.bfloat16),     # down projection, forward
                                            ((16384, 22016, 4096), False, torch.bfloat16),     # gate/up projection, forward
                                            ((16384, 11008, 4096), True, torch.bfloat16),      # dgrad of the down projection (N = 11008)
                                            ((4096, 4096, 16384), True, torch.float32),        # wgrad, contraction over 16384 tokens
                                            ((22016, 4096, 16384), True, torch.float32)])      # wgrad of gate/up
def test_config4_gemm_extents(ops, mnk, fused, out):
    m, n, k = mnk
    a, ae = _random_operand_dev(m, k, 1)
    b, be = _random_operand_dev(n, k, 2)
    asf, bsf = rm.to_blocked(ae.cpu()).cuda(), rm.to_blocked(be.cpu()).cuda()
    mask = None
    if fused:
        mask = torch.randint(0, 256, (m, n // 8), generator=torch.Generator(device="cuda").manual_seed(3), device="cuda", dtype=torch.uint8)
        mask |= torch.randint(0, 256, (m, n // 8), generator=torch.Generator(device="cuda").manual_seed(4), device="cuda", dtype=torch.uint8)
    alpha = 16.0 / 9.0
    d = ops.gemm_mxfp4_tn(a, asf, b, bsf, alpha, mask=mask, out_dtype=out)
    assert ops.device_status() == 0
    # (i) a row sample against float64 on the CPU: 128 rows spread over every 128-row tile position
    rows = torch.arange(0, m, m // 128) + torch.arange(128) % 128
    rows = rows.clamp(max=m - 1)
    ref = (_values(a[rows.cuda()], ae[rows.cuda()]) @ _values(b, be).T) * alpha
    if fused:
        mk = H.unpack_mask(mask[rows.cuda()])
        ref = rm.unrotate_mask(ref.float(), mk, rm.hadamard32()).double()
    err = _rel(d[rows.cuda()].cpu(), ref)
    print(mnk, "row sample vs float64:", err)
    assert err < (1e-5 if out == torch.float32 else 1e-2)
    # (ii) the whole product against an fp32 matmul of the de-quantized operands on the device
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    full = (ops.dequant(a, asf, 1.0, torch.float32) @ ops.dequant(b, bsf, 1.0, torch.float32).T) * alpha
    torch.backends.cuda.matmul.allow_tf32 = prev
    if fused:
        full = ops.unrotate_mask(full, mask, ops.HAD_SCALE_BF16)
    err = ((d.float() - full).norm() / full.norm()).item()
    print(mnk, "whole product vs fp32 matmul:", err)
    assert err < (1e-5 if out == torch.float32 else 1e-2)


# ------------------------------------------------------------------------------------------------
# the two-CTA kernel with a ragged last column tile
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("mnk", [(512, 1920, 640), (256, 1152, 256), (1024, 3456, 384)])
def test_two_cta_gemm_with_ragged_last_tile(ops, mnk):
    m, n, k = mnk  # N > 1024, N % 256 == 128, M % 256 == 0: the pair kernel with a half-empty last tile
    gen = torch.Generator().manual_seed(sum(mnk))
    a, ae, av = H.random_mxfp4(m, k, gen)
    b, be, bv = H.random_mxfp4(n, k, gen)
    dev = (a.cuda(), rm.to_blocked(ae).cuda(), b.cuda(), rm.to_blocked(be).cuda())
    ref = av.double() @ bv.double().T
    guard = torch.full((m + 2, n), float("nan"), device="cuda")
    d = guard[1:-1]
    ops.gemm_mxfp4_tn(*dev, alpha=1.0, out=d)
    assert _rel(d.cpu(), ref) < 1e-5
    assert bool(torch.isnan(guard[0]).all()) and bool(torch.isnan(guard[-1]).all())  # nothing written outside D
    mask = torch.rand(m, n, generator=gen) < 0.9
    pm = rm.Quantized(m, n, None, None, None, None, mask).packed_mask().cuda()
    ref_u = rm.unrotate_mask((ref * (16.0 / 9.0)).float(), mask, rm.hadamard32())
    d = ops.gemm_mxfp4_tn(*dev, alpha=16.0 / 9.0, mask=pm, out_dtype=torch.float32)
    assert _rel(d.cpu(), ref_u) < 1e-5
    d = ops.gemm_mxfp4_tn(*dev, alpha=16.0 / 9.0, mask=pm, out_dtype=torch.bfloat16)
    assert _rel(d.cpu().float(), ref_u) < 1e-2
    assert ops.device_status() == 0


# ------------------------------------------------------------------------------------------------
# exact ties
# ------------------------------------------------------------------------------------------------
def _tie_groups(n_groups, seed, integer_inputs):
    """Groups of 32 whose rotated values are small dyadic numbers, so that the rotation is exact in any
    summation order and many scaled values land exactly on a rounding tie.  H = 0.25 * Sylvester."""
    gen = torch.Generator().manual_seed(seed)
    if integer_inputs:  # sparse small integers: exactly representable in bf16
        x = torch.zeros(n_groups, 32)
        for _ in range(3):
            pos = torch.randint(0, 32, (n_groups,), generator=gen)
            x[torch.arange(n_groups), pos] += torch.randint(-12, 13, (n_groups,), generator=gen).float()
    else:  # x = t @ H^-1 for rotated targets t on a 0.25 grid
        t = torch.randint(-28, 29, (n_groups, 32), generator=gen).float() * 0.25
        sylv = torch.sign(rm.hadamard32(torch.float32))
        x = (t @ sylv) / 8.0
    return x


@pytest.mark.parametrize("dtype,integer_inputs", [(torch.float32, False), (torch.float32, True), (torch.bfloat16, True)])
def test_exact_ties_round_toward_the_smaller_magnitude(ops, dtype, integer_inputs):
    """|v| == 0.75, 1.75, 3.5 go DOWN like the reference's strict `>` ladder (mxfp4_triton.py:131-159); the
    hardware's round-to-nearest-even conversion alone would send them up."""
    h = torch.sign(rm.hadamard32(torch.float32)) * 0.25
    x = _tie_groups(128 * 128, 7, integer_inputs).reshape(128, -1)
    ref = rm.quant_fwd(x, h)
    v = (rm.rotate(x, h) / ref.shared.reshape(-1, 1)).abs().reshape(x.shape)
    ties = {t: int((v == t).sum()) for t in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)}
    print("exact ties in the constructed input:", ties)
    assert ties[0.75] > 50 and ties[1.75] > 50 and ties[3.5] > 50
    n_sf, n_code, n_mask, _, _ = _fwd_exceptions(ops, x, dtype=dtype, had_scale=0.25, h=h)
    print("exceptions on the tie input: scale groups", n_sf, "codes", n_code, "mask bits", n_mask)
    assert n_sf <= 2 and (n_code, n_mask) == (0, 0)  # a scale within an ulp of a power of two may differ; no code may
    assert ops.device_status() == 0
