"""The tcgen05 block-scaled MXFP4 GEMM against de-quantize-then-matmul in float64 on the CPU.

Tolerance (north-star): relative Frobenius error <= 1e-2.  With fp32 output the kernel is exact up
to fp32 accumulation order, so a much tighter 1e-5 is asserted there; bf16 output adds 2^-9 rounding.
"""
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


def _operands(m, n, k, seed):
    gen = torch.Generator().manual_seed(seed)
    a, ae, av = H.random_mxfp4(m, k, gen)
    b, be, bv = H.random_mxfp4(n, k, gen)
    return (a.cuda(), rm.to_blocked(ae).cuda(), b.cuda(), rm.to_blocked(be).cuda()), av, bv


@pytest.mark.parametrize("mnk", [(128, 128, 128), (128, 128, 256), (128, 256, 512), (256, 384, 640), (384, 1280, 1152),
                                 (256, 640, 2560), (1024, 512, 4096)])
def test_gemm_small_vs_cpu(ops, mnk):
    m, n, k = mnk
    dev, av, bv = _operands(m, n, k, seed=m + n + k)
    ref = av.double() @ bv.double().T
    d32 = ops.gemm_mxfp4_tn(*dev, alpha=1.0, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    err = ((d32.cpu().double() - ref).norm() / ref.norm()).item()
    print(mnk, "fp32 out rel err", err)
    assert err < 1e-5
    d16 = ops.gemm_mxfp4_tn(*dev, alpha=16.0 / 9.0, out_dtype=torch.bfloat16)
    err = ((d16.cpu().double() - ref * (16.0 / 9.0)).norm() / ref.norm()).item()
    assert err < 1e-2


def test_gemm_scale_extremes(ops):
    """Scales spanning the whole range the quantizers can emit, and zero groups."""
    gen = torch.Generator().manual_seed(9)
    a, ae, av = H.random_mxfp4(128, 256, gen, e_lo=100, e_hi=150)
    b, be, bv = H.random_mxfp4(256, 256, gen, e_lo=90, e_hi=135)
    ae[:, 0] = 0  # 2^-127: an all-zero group
    av[:, :32] = 0
    a[:, :16] = 0x88  # codes -0
    ref = av.double() @ bv.double().T
    d = ops.gemm_mxfp4_tn(a.cuda(), rm.to_blocked(ae).cuda(), b.cuda(), rm.to_blocked(be).cuda(), out_dtype=torch.float32)
    err = ((d.cpu().double() - ref).norm() / ref.norm()).item()
    assert err < 1e-5


def test_gemm_fused_mask_unrotate(ops):
    m, n, k = 256, 384, 512
    dev, av, bv = _operands(m, n, k, seed=77)
    gen = torch.Generator().manual_seed(78)
    mask = torch.rand(m, n, generator=gen) < 0.95
    q = rm.Quantized(m, n, None, None, None, None, mask)
    acc = (av.double() @ bv.double().T * (16.0 / 9.0)).float()
    ref = rm.unrotate_mask(acc, mask, rm.hadamard32())
    d = ops.gemm_mxfp4_tn(*dev, alpha=16.0 / 9.0, mask=q.packed_mask().cuda(), had_scale=ops.HAD_SCALE_BF16,
                          out_dtype=torch.float32)
    err = ((d.cpu() - ref).norm() / ref.norm()).item()
    assert err < 1e-5
    d = ops.gemm_mxfp4_tn(*dev, alpha=16.0 / 9.0, mask=q.packed_mask().cuda(), out_dtype=torch.bfloat16)
    assert ((d.cpu().float() - ref).norm() / ref.norm()).item() < 1e-2


def test_gemm_full_size_linearity_and_torch_reference(ops):
    """At a 7B-layer shape: compare with a torch fp32 matmul of the de-quantized operands on the
    GPU, and check linearity in alpha (a size-independent property)."""
    m, n, k = 4096, 4096, 4096
    gen = torch.Generator().manual_seed(5)
    a, ae, _ = H.random_mxfp4(m, k, gen)
    b, be, _ = H.random_mxfp4(n, k, gen)
    a, b, asf, bsf = a.cuda(), b.cuda(), rm.to_blocked(ae).cuda(), rm.to_blocked(be).cuda()
    d1 = ops.gemm_mxfp4_tn(a, asf, b, bsf, alpha=1.0, out_dtype=torch.float32)
    d2 = ops.gemm_mxfp4_tn(a, asf, b, bsf, alpha=2.0, out_dtype=torch.float32)
    assert bool((d2 == 2 * d1).all())
    av = ops.dequant(a, asf, 1.0, torch.float32)
    bv = ops.dequant(b, bsf, 1.0, torch.float32)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = av @ bv.T
    torch.backends.cuda.matmul.allow_tf32 = prev
    err = ((d1 - ref).norm() / ref.norm()).item()
    print("4096^3 rel err vs torch fp32", err)
    assert err < 1e-5
    assert ops.device_status() == 0


def test_layer_against_golden(ops, golden_dir):
    """Whole QuantizedLinear forward + backward on the golden layer: forward codes identical to the
    reference's quantized operands, GEMM outputs within 1e-2 of the reference's y / dx / dw when the
    reference's own tl.rand seeds are replayed."""
    import os

    import numpy as np

    g = np.load(os.path.join(golden_dir, "linear_fwd_bwd.npz"))
    x, w, e = (torch.from_numpy(g[k]) for k in "xwe")
    signs = int(g["signs"])
    seeds = [int(s) for s in g["seeds"]]
    xd, wd, ed = x.bfloat16().cuda(), w.bfloat16().cuda(), e.bfloat16().cuda()
    xc, xs, xm = ops.quant_fwd(xd)
    wc, ws, wm = ops.quant_fwd(wd)
    y = ops.gemm_mxfp4_tn(xc, xs, wc, ws, 1.0, out_dtype=torch.float32).cpu()
    yr = torch.from_numpy(g["y"])
    assert ((y - yr).norm() / yr.norm()).item() < 1e-5
    a = ops.SR_OPERAND_SCALE ** 2
    R = ops.ROUND_SR_TLRAND
    ec, es = ops.quant_bwd(ed, signs=signs, rounding=R, seed=seeds[0])
    wtc, wts = ops.requant_t(wc, ws, signs=signs, rounding=R, seed=seeds[1])
    dx = ops.gemm_mxfp4_tn(ec, es, wtc, wts, a, mask=xm, out_dtype=torch.float32).cpu()
    etc_, ets = ops.quant_bwd_t(ed, signs=signs, rounding=R, seed=seeds[2])
    xtc, xts = ops.requant_t(xc, xs, signs=signs, rounding=R, seed=seeds[3])
    dw = ops.gemm_mxfp4_tn(etc_, ets, xtc, xts, a, mask=wm, out_dtype=torch.float32).cpu()
    for name, got in (("dx", dx), ("dw", dw)):
        ref = torch.from_numpy(g[name])
        err = ((got - ref).norm() / ref.norm()).item()
        print(name, "rel err vs reference", err)
        assert err < 1e-5


@pytest.mark.parametrize("owners", [1, 2, 4, 8])
def test_gemm_scatter_equals_dense_result_and_shard_reduce_is_ordered(ops, owners):
    """The scattered store (one GPU standing in for every owner) lands exactly the rows of the dense fp32
    result in each owner's slot, with the fused mask + un-rotation; the slot sum is the in-order sum."""
    m, n, k = 512, 768, 1024
    dev, av, bv = _operands(m, n, k, seed=91)
    gen = torch.Generator().manual_seed(92)
    mask = torch.rand(m, n, generator=gen) < 0.9
    pm = rm.Quantized(m, n, None, None, None, None, mask).packed_mask().cuda()
    dense = ops.gemm_mxfp4_tn(*dev, alpha=16.0 / 9.0, mask=pm, had_scale=ops.HAD_SCALE_BF16, out_dtype=torch.float32)
    rpo = m // owners
    slots = torch.full((owners, rpo, n), float("nan"), device="cuda")
    ops.gemm_mxfp4_tn_scatter(*dev, [slots[o].data_ptr() for o in range(owners)], rpo, alpha=16.0 / 9.0, mask=pm,
                              had_scale=ops.HAD_SCALE_BF16)
    assert torch.equal(slots.reshape(m, n), dense)
    out = torch.empty(rpo, n, device="cuda")
    ops.shard_reduce(slots.data_ptr(), owners, rpo * n, 1.0 / owners, out)
    acc = slots[0].clone()
    for o in range(1, owners):
        acc = acc + slots[o]
    assert torch.equal(out, acc * (1.0 / owners))
    assert ops.device_status() == 0


def test_gemm_scatter_rejects_bad_splits(ops):
    dev, _, _ = _operands(512, 256, 256, seed=93)
    buf = torch.empty(512, 256, device="cuda")
    with pytest.raises(ValueError):
        ops.gemm_mxfp4_tn_scatter(*dev, [buf.data_ptr()] * 3, 160)        # 3 * 160 != 512
    with pytest.raises(ValueError):
        ops.gemm_mxfp4_tn_scatter(*dev, [buf.data_ptr()] * 16, 32)        # more than 8 owners
    with pytest.raises(ValueError):
        ops.gemm_mxfp4_tn_scatter(*dev, [buf.data_ptr(), 0], 256)         # NULL owner
