"""The reference-facing boundary on the GPU: the `quartet_b200::*` custom operators (eager, traced and
compiled), the three MXFP4 registry entries in every configuration the reference's flags can produce
(general rotations, deterministic rounding, the 1.009276 re-scaling), the other two backward schemes, the
rotation-free quantizer of the post-training tools and the weight export -- each against the CPU oracle."""
import random

import numpy as np
import pytest
import torch

from oracle import ref_math as rm
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Q():
    import __graft_entry__ as entry

    entry.build()
    import quartet_b200.quantization as q

    return q


@pytest.fixture(scope="module")
def ops(Q):
    from quartet_b200 import ops

    return ops


def _production_linear(Q, k, n, **gkw):
    return Q.QuantizedLinear(
        k, n, bias=False,
        weight_quantizer=Q.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
        activation_quantizer=Q.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
        gradient_quantizer=Q.QUANTIZER_CLASSES["AlbertTsengQuantizer"](**gkw),
        backward_scheme=Q.BACKWARD_SCHEMES["Q(E)Q(Wt)t_Q(Et)Q(Xt)t"](),
    ).cuda()


# ------------------------------------------------------------------------------------------------
# custom operators
# ------------------------------------------------------------------------------------------------
def test_operators_equal_the_direct_calls_and_pass_opcheck(ops):
    import quartet_b200.torch_ops  # noqa: F401  (registers the operators)

    t = torch.ops.quartet_b200
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(256, 384, generator=g, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(128, 384, generator=g, device="cuda", dtype=torch.bfloat16)
    xc, xs, xm = t.quant_fwd(x, ops.HAD_SCALE_BF16, ops.QUEST_GAUSSIAN_SCALE)
    for got, want in zip((xc, xs, xm), ops.quant_fwd(x)):
        assert torch.equal(got, want)
    wc, ws, _ = t.quant_fwd(w, ops.HAD_SCALE_BF16, ops.QUEST_GAUSSIAN_SCALE)
    y = t.gemm_mxfp4_tn(xc, xs, wc, ws, 1.0, None, ops.HAD_SCALE_BF16, torch.float32)
    assert torch.equal(y, ops.gemm_mxfp4_tn(xc, xs, wc, ws, 1.0, out_dtype=torch.float32))
    ec, es = t.quant_bwd(x, ops.HAD_SCALE_BF16, 5, None, 1, 7, 0, None)
    assert torch.equal(ec, ops.quant_bwd(x, signs=5, seed=7)[0])
    tc, ts = t.quant_bwd_t(x, ops.HAD_SCALE_BF16, 5, None, 1, 7, 0, None)
    d = t.quant_bwd_dual(x, ops.HAD_SCALE_BF16, 5, None, 1, 7, 7, 0)
    assert torch.equal(d[0], ec) and torch.equal(d[2], tc) and torch.equal(d[3], ts)
    rc, rs = t.requant_t(xc, xs, 1.0, ops.HAD_SCALE_BF16, 0, None, 0, 0, 0, None)
    assert rc.shape == (384, 128) and torch.equal(rc, ops.requant_t(xc, xs, rounding=0)[0])
    assert torch.equal(t.dequant(xc, xs, 1.0, torch.float32), ops.dequant(xc, xs))
    assert torch.equal(t.unrotate_mask(y, None, ops.HAD_SCALE_BF16, torch.float32), ops.unrotate_mask(y, None))
    # fake kernels agree with the real ones on shapes, dtypes and strides; schemas are consistent
    for op, args in ((t.quant_fwd.default, (x, ops.HAD_SCALE_BF16, ops.QUEST_GAUSSIAN_SCALE)),
                     (t.quant_bwd_dual.default, (x, ops.HAD_SCALE_BF16, 0, None, 0, 0, 0, 0)),
                     (t.requant_t.default, (xc, xs, 1.0, ops.HAD_SCALE_BF16, 0, None, 0, 0, 0, None)),
                     (t.gemm_mxfp4_tn.default, (xc, xs, wc, ws, 1.0, xm[:, :16].contiguous(), ops.HAD_SCALE_BF16, torch.bfloat16))):
        torch.library.opcheck(op, args, test_utils=("test_schema", "test_faketensor"))


def _grads(lin, x, e):
    lin.weight.grad = None
    xx = x.clone().requires_grad_(True)
    y = lin(xx)
    y.backward(e)
    return y.detach(), xx.grad, lin.weight.grad.clone()


def test_layer_operator_equals_the_autograd_function_and_compiles(Q, ops, monkeypatch):
    """The custom-operator route of QuantizedLinear (what a compiled model runs) gives the bits of the eager
    autograd function (deterministic rounding, same sign draws), and `torch.compile(fullgraph=True)` traces the
    layer without a break."""
    torch.manual_seed(3)
    lin = _production_linear(Q, 256, 384, stochastic=False, rerotate="signs")
    x = torch.randn(4, 64, 256, device="cuda", dtype=torch.bfloat16)
    e = torch.randn(4, 64, 384, device="cuda", dtype=torch.bfloat16) * 1e-3

    torch.manual_seed(11)
    y1, dx1, dw1 = _grads(lin, x, e)  # eager: the plain autograd function (also what the multi-GPU sink path uses)
    # the same layer through the pair of custom operators, called eagerly
    lin.backward_scheme.g_quantizer._signs_dev = None
    lin.backward_scheme.g_quantizer._signs_host = 0
    from quartet_b200 import torch_ops

    def via_operator(self, xin):
        return torch_ops.quantized_linear(xin, self.weight, self._handle, xin.dtype)

    torch.manual_seed(11)
    with monkeypatch.context() as m:
        m.setattr(Q.QuantizedLinear, "forward", via_operator)
        y2, dx2, dw2 = _grads(lin, x, e)
    assert torch.equal(y1, y2) and torch.equal(dx1, dx2) and torch.equal(dw1, dw2)

    # compiled: one graph, no break
    lin.backward_scheme.g_quantizer._signs_dev = None
    torch._dynamo.reset()
    clin = torch.compile(lin, fullgraph=True)
    torch.manual_seed(11)
    lin.weight.grad = None
    xx = x.clone().requires_grad_(True)
    y3 = clin(xx)
    y3.backward(e)
    assert torch.equal(y3.detach(), y1) and torch.equal(xx.grad, dx1) and torch.equal(lin.weight.grad, dw1)
    assert ops.device_status() == 0


def test_compiled_model_under_autocast_trains(Q, ops):
    """`torch.compile(model)` with bf16 autocast around forward and backward, as the reference's training loop
    runs it (src/optim/base.py:38-50, 190-200): no graph-break error, loss falls, gradients match eager closely."""
    import copy

    from tests.llama_harness import TinyLlama

    torch.manual_seed(5)
    gkw = {"stochastic": False, "rerotate": None}
    eager = TinyLlama(Q, gkw=gkw).cuda()
    comp_src = copy.deepcopy(eager)
    torch._dynamo.reset()
    compiled = torch.compile(comp_src)
    idx = torch.randint(0, 512, (4, 128), device="cuda")
    tgt = torch.roll(idx, -1, 1)

    def step(model, params):
        for p in params:
            p.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(idx, tgt)
            loss.backward()
        return loss

    l_e = step(eager, eager.parameters())
    l_c = step(compiled, comp_src.parameters())
    assert abs(l_e.item() - l_c.item()) < 2e-2 * abs(l_e.item())
    for (n, a), (_, b) in zip(eager.named_parameters(), comp_src.named_parameters()):
        cos = torch.nn.functional.cosine_similarity(a.grad.flatten().float(), b.grad.flatten().float(), dim=0).item()
        assert cos > 0.85, (n, cos)  # inductor fuses the norms and activations differently: some quantization decisions flip
    opt = torch.optim.AdamW(comp_src.parameters(), lr=3e-3)
    losses = []
    for _ in range(15):
        losses.append(step(compiled, comp_src.parameters()).item())
        opt.step()
    assert losses[-1] < 0.8 * losses[0]
    assert ops.device_status() == 0


# ------------------------------------------------------------------------------------------------
# the three MXFP4 registry entries, every configuration
# ------------------------------------------------------------------------------------------------
def _sylv(n):
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (h * n ** -0.5).float()


def test_aligned_quantizer_matches_oracle(Q, ops):
    """AlignedAlbertTsengQuantizer (mxfp4.py:95-124): absmax scale, round to nearest, output x 1.009276."""
    g = torch.Generator().manual_seed(1)
    x = H.bf16r(torch.randn(256, 256, generator=g) * 1e-2)
    q = Q.QUANTIZER_CLASSES["AlignedAlbertTsengQuantizer"]()
    out = q(x.bfloat16().cuda()).float().cpu()
    ref = (rm.quant_bwd(x, rm.hadamard32(), None, stochastic=False).dequant().bfloat16() * 1.009276).float()
    assert torch.equal(out, ref)
    # and the plain quantizer with stochastic=False is the same without the factor
    q2 = Q.QUANTIZER_CLASSES["AlbertTsengQuantizer"](stochastic=False)
    out2 = q2(x.cuda()).cpu()  # fp32 input: the rotation matrix stays fp32
    ref2 = rm.quant_bwd(x, rm.hadamard32(torch.float32), None, stochastic=False).dequant()
    bad = out2 != ref2
    print("fp32 round-to-nearest absmax quantizer: elements differing from the oracle", int(bad.sum()))
    assert int(bad.sum()) <= 2
    # straight-through backward: grad @ H^T
    xg = x.bfloat16().cuda().requires_grad_(True)
    go = torch.randn(256, 256, generator=torch.Generator().manual_seed(2)).bfloat16()
    q(xg).backward(go.cuda())
    ref_g = (go.float().reshape(-1, 32) @ rm.hadamard32().T).reshape(256, 256)
    assert ((xg.grad.float().cpu() - ref_g).norm() / ref_g.norm()).item() < 1e-2


@pytest.mark.parametrize("dim", [32, 64, 128])
def test_general_rotations(Q, ops, dim):
    """hadamard_dim 64 / 128 and a dense orthogonal matrix (rerotate="O32"): rotation by matmul, the rest by the
    rotation-free kernel; against the oracle fed the same matrix and the same tl.rand stream."""
    g = torch.Generator().manual_seed(dim)
    x = H.bf16r(torch.randn(128, 512, generator=g) * 3e-3)
    q = Q.QUANTIZER_CLASSES["AlbertTsengQuantizer"](hadamard_dim=dim, stochastic=True, rerotate="O32")
    q.sr_rounding = ops.ROUND_SR_TLRAND
    xd = x.bfloat16().cuda()
    mats = [None, "O32"]
    for kind in mats:
        if kind == "O32":
            torch.manual_seed(99)
            q._see(xd)
            q.re_randomize(device="cuda")
            assert not q.is_builtin_rotation
        hm = q.hadamard_matrix
        if kind is None:
            q._see(xd)
            hm = q.hadamard_matrix
            assert torch.equal(hm.float().cpu(), _sylv(dim).bfloat16().float())
        else:
            eye = (hm.float() @ hm.float().T).cpu()
            assert (eye - torch.eye(dim)).abs().max() < 2e-2  # orthogonal up to bf16 rounding of its entries
        random.seed(4)
        seed = random.randint(0, 1000000)
        random.seed(4)
        out = q(xd).float().cpu()
        u = rm.triton_rand(seed, np.arange(x.numel())).reshape(x.shape)
        ref = rm.quant_bwd(x, hm.float().cpu(), u).dequant().bfloat16().float()
        bad = out != ref
        print(f"dim {dim} {kind}: elements differing from the oracle {int(bad.sum())} of {x.numel()}")
        # the device matmul sums the rotation in another order than the CPU: last-ulp differences flip a few decisions
        assert int(bad.sum()) <= 6
    # forward (std-scaled) quantizer with a 64-point rotation, and its straight-through backward
    if dim == 64:
        fq = Q.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](hadamard_dim=64)
        xg = xd.clone().requires_grad_(True)
        y = fq(xg)
        h64 = _sylv(64).bfloat16().float()
        ref = rm.quant_fwd(x, h64)
        bad = y.detach().float().cpu() != ref.dequant()
        assert int(bad.sum()) <= 6
        go = torch.ones_like(y)
        y.backward(go)
        ref_g = ((go.float().cpu() * ref.mask).reshape(-1, 64) @ h64.T).reshape(x.shape)
        assert ((xg.grad.float().cpu() - ref_g).norm() / ref_g.norm()).item() < 1e-2
    assert ops.device_status() == 0


def test_layer_with_general_rotation_composes(Q, ops):
    """A gradient quantizer with rerotate="O32" sends the layer down the composed path; it still runs on this
    library's kernels (packed operands, MXFP4 GEMMs) and gives gradients close to the plain ones."""
    torch.manual_seed(8)
    lin = _production_linear(Q, 256, 256, stochastic=True, rerotate="O32")
    x = torch.randn(256, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    e = torch.randn(256, 256, device="cuda", dtype=torch.bfloat16) * 1e-2
    with torch.autocast("cuda", dtype=torch.bfloat16):  # fp32 master weights, bf16 activations, as in training
        y = lin(x)
        y.backward(e)
    assert not lin.backward_scheme.g_quantizer.is_builtin_rotation
    dx_ref = e.float() @ lin.weight.float()
    dw_ref = e.float().T @ x.float()
    assert torch.nn.functional.cosine_similarity(x.grad.float().flatten(), dx_ref.flatten(), dim=0) > 0.9
    assert torch.nn.functional.cosine_similarity(lin.weight.grad.float().flatten(), dw_ref.flatten(), dim=0) > 0.9


# ------------------------------------------------------------------------------------------------
# the other two backward schemes
# ------------------------------------------------------------------------------------------------
def test_half_quantized_scheme_against_oracle(Q, ops):
    """"Q(E)W_Q(Et)X" (backward.py:21-45): dX = Q(E) W, dW = Q(E^T) X with deterministic rounding, vs the oracle."""
    g = torch.Generator().manual_seed(12)
    x = H.bf16r(torch.randn(256, 128, generator=g))
    w = H.bf16r(torch.randn(384, 128, generator=g) * 0.05)
    e = H.bf16r(torch.randn(256, 384, generator=g) * 1e-2)
    lin = Q.QuantizedLinear(128, 384, bias=False, gradient_quantizer=Q.AlbertTsengQuantizer(stochastic=False),
                            backward_scheme=Q.BACKWARD_SCHEMES["Q(E)W_Q(Et)X"]()).cuda().bfloat16()
    with torch.no_grad():
        lin.weight.copy_(w)
    xd = x.bfloat16().cuda().requires_grad_(True)
    lin(xd).backward(e.bfloat16().cuda())
    h = rm.hadamard32()
    qe = rm.quant_bwd(e, h, None, stochastic=False).dequant().bfloat16().float()
    qet = rm.quant_bwd(e.T.contiguous(), h, None, stochastic=False).dequant().bfloat16().float()
    dx_ref, dw_ref = qe @ w, qet @ x
    assert ((xd.grad.float().cpu() - dx_ref).norm() / dx_ref.norm()).item() < 1e-2
    assert ((lin.weight.grad.float().cpu() - dw_ref).norm() / dw_ref.norm()).item() < 1e-2
    # plain scheme: autograd's own gradients
    lin2 = Q.QuantizedLinear(128, 384, bias=False, backward_scheme=Q.BACKWARD_SCHEMES["EW_EtX"]()).cuda().bfloat16()
    with torch.no_grad():
        lin2.weight.copy_(w)
    xd2 = x.bfloat16().cuda().requires_grad_(True)
    lin2(xd2).backward(e.bfloat16().cuda())
    assert ((xd2.grad.float().cpu() - e @ w).norm() / (e @ w).norm()).item() < 1e-2


def test_fully_quantized_scheme_composed_equals_fused(Q, ops, monkeypatch):
    """The composed "Q(E)Q(Wt)t_Q(Et)Q(Xt)t" path (quantizer modules + packed backward GEMMs) against the oracle's
    layer with deterministic rounding."""
    g = torch.Generator().manual_seed(13)
    x = H.bf16r(torch.randn(256, 256, generator=g))
    w = H.bf16r(torch.randn(128, 256, generator=g) * 0.05)
    e = H.bf16r(torch.randn(256, 128, generator=g) * 1e-2)
    lin = _production_linear(Q, 256, 128, stochastic=False, rerotate=None).bfloat16()
    with torch.no_grad():
        lin.weight.copy_(w)
    monkeypatch.setattr(Q.QuantizedLinear, "_fusable", lambda self, x_: False)
    xd = x.bfloat16().cuda().requires_grad_(True)
    y = lin(xd)
    y.backward(e.bfloat16().cuda())
    h = rm.hadamard32()
    y_ref, xq, wq = rm.linear_forward(x, w, h)
    qs = [rm.quant_bwd(t, h, None, stochastic=False) for t in
          (e, wq.dequant().T.contiguous(), e.T.contiguous(), xq.dequant().T.contiguous())]
    dx_ref = rm.unrotate_mask(qs[0].dequant() @ qs[1].dequant().T, xq.mask, h)
    dw_ref = rm.unrotate_mask(qs[2].dequant() @ qs[3].dequant().T, wq.mask, h)
    assert ((y.float().cpu() - y_ref).norm() / y_ref.norm()).item() < 1e-2
    assert ((xd.grad.float().cpu() - dx_ref).norm() / dx_ref.norm()).item() < 1e-2
    assert ((lin.weight.grad.float().cpu() - dw_ref).norm() / dw_ref.norm()).item() < 1e-2


# ------------------------------------------------------------------------------------------------
# rotation-free quantizer and weight export
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rotation_free_quantizer_matches_oracle(ops, dtype):
    """quartet_quant_group32: the std-scaled and the absmax-scaled quantizer without rotation
    (src/quarot_utils/mxfp4_quant_utils.py:24-113 is this with round-to-nearest), vs the oracle with H = identity."""
    g = torch.Generator().manual_seed(21)
    x = H.bf16r(torch.randn(300, 256, generator=g))
    eye = torch.eye(32)
    xd = x.to(dtype).cuda()
    codes, sf, mask = ops.quant_group32(xd, 0)
    ref = rm.quant_fwd(x, eye)
    idx, neg = H.unpack_codes(codes)
    n_sf, n_code, _ = H.compare_quantized(idx, neg, H.unpack_sf(sf, 300, 256), ref)
    mask_bad = int((H.unpack_mask(mask) != ref.mask).sum())
    print("rotation-free std-scaled: scale groups", n_sf, "codes", n_code, "mask bits", mask_bad)
    assert n_sf <= 1 and n_code <= 2 and mask_bad <= 40  # the group moments are summed in another order: a scale can sit on a power of two
    u = torch.rand(300, 256, generator=g)
    for rounding, noise, stoch in ((ops.ROUND_NEAREST, None, False), (ops.ROUND_SR_NOISE, u, True)):
        codes, sf, _ = ops.quant_group32(xd, 1, rounding=rounding, noise=None if noise is None else noise.cuda())
        ref = rm.quant_bwd(x, eye, noise, stochastic=stoch)
        idx, neg = H.unpack_codes(codes)
        assert H.compare_quantized(idx, neg, H.unpack_sf(sf, 300, 256), ref)[:2] == (0, 0)
    assert ops.device_status() == 0


def test_exported_weight_matches_oracle(Q, ops):
    """export_mxfp4: codes and blocked scales of the forward-quantized weight, bit for bit the oracle's."""
    g = torch.Generator().manual_seed(31)
    w = torch.randn(384, 256, generator=g) * 0.02
    lin = _production_linear(Q, 256, 384)
    with torch.no_grad():
        lin.weight.copy_(w)
    codes, sf, had_scale = lin.export_mxfp4()
    ref = rm.quant_fwd(w, rm.hadamard32(torch.float32))  # fp32 master weights: the rotation matrix stays fp32
    assert abs(had_scale - float(rm.hadamard32(torch.float32)[0, 0])) < 1e-9
    idx, neg = H.unpack_codes(codes)
    n_sf, n_code, _ = H.compare_quantized(idx, neg, H.unpack_sf(sf, 384, 256), ref)
    assert (n_sf, n_code) == (0, 0)
    assert torch.equal(sf.cpu(), rm.to_blocked(ref.e8m0))
