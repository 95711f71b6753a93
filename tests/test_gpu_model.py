"""Model-level use of the drop-in package: a small Llama-style decoder whose block linears are
QuantizedLinear (production quantizer / scheme names), bf16 autocast around forward AND backward as
the reference's training loop does (src/optim/base.py:190-200)."""
import copy

import pytest
import torch

from tests.llama_harness import TinyLlama

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Q():
    import __graft_entry__ as entry

    entry.build()
    import quartet_b200.quantization as q

    return q


def _step(model, idx, tgt):
    for p in model.parameters():
        p.grad = None
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = model(idx, tgt)
        loss.backward()
    return loss


def test_fused_path_matches_composed_modules_at_model_level(Q, monkeypatch):
    torch.manual_seed(0)
    gkw = {"stochastic": False, "rerotate": "signs"}  # deterministic rounding so both paths are comparable
    fused = TinyLlama(Q, gkw=gkw).cuda()
    composed = copy.deepcopy(fused)
    idx = torch.randint(0, 512, (4, 128), device="cuda")
    tgt = torch.randint(0, 512, (4, 128), device="cuda")
    l1 = _step(fused, idx, tgt)
    monkeypatch.setattr(Q.QuantizedLinear, "_fusable", lambda self, x: False)  # compose quantizer modules + F.linear
    l2 = _step(composed, idx, tgt)
    assert abs(l1.item() - l2.item()) < 2e-2 * abs(l2.item())
    for (n1, p1), (_, p2) in zip(fused.named_parameters(), composed.named_parameters()):
        assert p1.grad is not None and torch.isfinite(p1.grad).all(), n1
        cos = torch.nn.functional.cosine_similarity(p1.grad.flatten().float(), p2.grad.flatten().float(), dim=0).item()
        assert cos > 0.98, (n1, cos)


def test_training_reduces_loss(Q):
    from quartet_b200 import ops

    torch.manual_seed(1)
    model = TinyLlama(Q).cuda()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    idx = torch.randint(0, 512, (8, 128), device="cuda")
    tgt = torch.roll(idx, -1, 1)
    losses = []
    for _ in range(30):
        losses.append(_step(model, idx, tgt).item())
        opt.step()
    print("loss", losses[0], "->", losses[-1])
    assert losses[-1] < 0.7 * losses[0]
    assert list(model.blocks[0].c_attn.state_dict().keys()) == ["weight"]
    assert ops.device_status() == 0


def test_grouped_query_block_trains_and_exports_weights(Q):
    """Llama-3 style grouped-query attention (4 query heads, 2 key/value heads: qkv is 512 + 2 * 256 wide)
    and the MXFP4 export of a trained layer's weight."""
    from quartet_b200 import ops

    torch.manual_seed(2)
    model = TinyLlama(Q, d=512, n_head=4, n_kv_head=2, n_layer=1).cuda()
    assert model.blocks[0].c_attn.out_features == 1024
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    idx = torch.randint(0, 512, (4, 128), device="cuda")
    tgt = torch.roll(idx, -1, 1)
    losses = []
    for _ in range(20):
        losses.append(_step(model, idx, tgt).item())
        opt.step()
    assert losses[-1] < 0.8 * losses[0]
    lin = model.blocks[0].c_attn
    codes, sf, had_scale = lin.export_mxfp4()
    assert codes.shape == (1024, 256) and codes.dtype == torch.uint8 and sf.numel() == ops.sf_bytes(1024, 512)
    # the exported operand reproduces the layer's forward: y = Q(x) . export^T
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        want = lin(x)
    xc, xs, _ = ops.quant_fwd(x, lin.activation_quantizer.had_scale, ops.QUEST_GAUSSIAN_SCALE, return_mask=False)
    y = ops.gemm_mxfp4_tn(xc, xs, codes, sf, 1.0, out_dtype=torch.bfloat16)
    assert torch.equal(y, want)


@pytest.mark.skipif(__import__("tests.ref_model", fromlist=["x"]).reference_src() is None,
                    reason="needs a reference checkout on the GPU machine: set QUARTET_REF to its `src` directory")
@pytest.mark.parametrize("compiled", [False, True])
def test_reference_llama_trains_on_this_package(Q, compiled):
    """The reference's own 30M Llama (src/models/llama.py:176-262, unchanged), its block linears served by this
    package, one training step with bf16 autocast around forward and backward (src/optim/base.py:190-200), eager and
    under torch.compile (src/optim/base.py:38-40)."""
    from quartet_b200 import ops
    from tests.ref_model import reference_on_this_package

    with reference_on_this_package() as (llama, args):
        torch.manual_seed(0)
        model = llama.Llama(args).cuda()
        step_model = torch.compile(model) if compiled else model
        idx = torch.randint(0, 32000, (4, 512), device="cuda")
        tgt = torch.randint(0, 32000, (4, 512), device="cuda")
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
        losses = []
        for _ in range(3):
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = step_model(idx, targets=tgt)["loss"]
                loss.backward()
            opt.step()
            losses.append(loss.item())
        assert abs(losses[0] - 10.37) < 0.5 and losses[-1] < losses[0]  # ln(32000) at initialisation, falling on a fixed batch
        for n, p in model.named_parameters():
            assert p.grad is not None and torch.isfinite(p.grad).all(), n
        assert ops.device_status() == 0


@pytest.mark.parametrize("fuse_producers", [False, True])
def test_training_step_matches_the_reference_models_own_step(Q, golden_dir, fuse_producers):
    """(fuse_producers: the norms and the SwiGLU product computed inside the forward quantizers,
    Q.rmsnorm_linear / Q.swiglu_linear, held to the same comparison: their backward runs the operations autograd
    runs for the unfused steps, in the same order, and on this input reproduces the unfused gradients bit for bit.)
    tests/golden/llama_tiny_step.npz holds one fp32 training step of the REFERENCE'S OWN Llama (its model code,
    its quantization package, its kernel under the Triton interpreter; generator: tests/golden/make_model_golden.py).
    The harness model with the same parameters, its block linears served by this library, must reproduce the loss,
    the logits and every parameter's gradient.  Rounding is to nearest in the gradient quantizer, so nothing is
    random; what differs is fp32 summation order (and the quantization decisions that flips)."""
    import os

    import numpy as np

    from quartet_b200 import ops

    g = np.load(os.path.join(golden_dir, "llama_tiny_step.npz"))
    model = TinyLlama(Q, vocab=256, d=128, n_layer=2, n_head=1, multiple_of=256, gkw={"stochastic": False},
                      eps=float(g["rmsnorm_eps"]), fuse_producers=fuse_producers).cuda()
    assert model.blocks[0].hidden == 512

    def ref_name(n):  # harness parameter name -> the reference model's
        n = n.replace("blocks.", "transformer.h.").replace(".ln1.", ".ln_1.").replace(".ln2.", ".ln_2.")
        n = n.replace(".c_attn.", ".attn.c_attn.").replace(".attn_proj.", ".attn.c_proj.").replace(".w12.", ".mlp.w12.")
        if ".c_proj." in n and ".attn." not in n:
            n = n.replace(".c_proj.", ".mlp.c_proj.")
        return {"wte.weight": "transformer.wte.weight", "ln_f.weight": "transformer.ln_f.weight"}.get(n, n)

    with torch.no_grad():
        for n, p in model.named_parameters():
            bits = torch.from_numpy(g["param:" + ref_name(n)])
            p.copy_(bits.view(torch.bfloat16).float().reshape(p.shape))
    idx, tgt = torch.from_numpy(g["idx"]).cuda(), torch.from_numpy(g["targets"]).cuda()
    loss, logits = model(idx, tgt, return_logits=True)  # fp32 throughout, like the golden run
    loss.backward()
    print("loss", loss.item(), "reference", float(g["loss"]))
    assert abs(loss.item() - float(g["loss"])) < 1e-4
    ref_logits = torch.from_numpy(g["logits_sample"])
    err = ((logits[:, ::8, :].float().cpu() - ref_logits).norm() / ref_logits.norm()).item()
    print("logits rel err", err)
    assert err < 1e-4
    worst = (1.0, "")
    for n, p in model.named_parameters():
        rn = ref_name(n)
        gn = float(g["gnorm:" + rn])
        row = torch.from_numpy(g["grow:" + rn])
        mine = p.grad.float().cpu()
        assert abs(mine.norm().item() - gn) < 2e-3 * gn, (n, mine.norm().item(), gn)
        got_row = mine.reshape(mine.shape[0], -1)[0] if mine.dim() > 1 else mine
        if row.norm().item() == 0.0:  # e.g. the embedding row of a token that does not occur in the batch
            assert got_row.norm().item() == 0.0, n
            continue
        cos = torch.nn.functional.cosine_similarity(got_row, row, dim=0).item()
        worst = min(worst, (cos, n))
        assert cos > 0.9999, (n, cos)
    print("lowest first-row cosine", worst)
    assert ops.device_status() == 0


@pytest.mark.parametrize("compiled", [False, True])
def test_producer_fused_blocks_match_the_plain_blocks(Q, compiled):
    """The harness model with RMSNorm and SwiGLU computed inside the forward quantizers of the layers they feed
    against the same model with the steps as torch operations, bf16 autocast, round-to-nearest gradients: the same
    loss and gradients up to the quantization decisions that the last place of the norm's row statistic flips;
    and the fused form traces under torch.compile and trains."""
    from quartet_b200 import ops

    torch.manual_seed(7)
    gkw = {"stochastic": False, "rerotate": None}
    plain = TinyLlama(Q, gkw=gkw).cuda()
    fused = TinyLlama(Q, gkw=gkw, fuse_producers=True).cuda()
    fused.load_state_dict(plain.state_dict())
    with torch.no_grad():  # norm weights away from 1 so that their gradients and their use are both exercised
        for m in (plain, fused):
            torch.manual_seed(8)
            for blk in m.blocks:
                blk.ln1.weight.add_(0.1 * torch.randn_like(blk.ln1.weight))
                blk.ln2.weight.add_(0.1 * torch.randn_like(blk.ln2.weight))
    idx = torch.randint(0, 512, (4, 128), device="cuda")
    tgt = torch.roll(idx, -1, 1)
    runner = fused
    if compiled:
        torch._dynamo.reset()
        runner = torch.compile(fused)
    l_p = _step(plain, idx, tgt)
    for p in fused.parameters():
        p.grad = None
    with torch.autocast("cuda", dtype=torch.bfloat16):
        l_f = runner(idx, tgt)
        l_f.backward()
    print("loss plain", l_p.item(), "fused", l_f.item())
    assert abs(l_p.item() - l_f.item()) < 2e-3 * abs(l_p.item())
    for (n, a), (_, b) in zip(plain.named_parameters(), fused.named_parameters()):
        assert b.grad is not None and torch.isfinite(b.grad).all(), n
        cos = torch.nn.functional.cosine_similarity(a.grad.flatten().float(), b.grad.flatten().float(), dim=0).item()
        # compiled: inductor evaluates the surrounding bf16 operations in another order, and some 4-bit decisions flip
        assert cos > (0.85 if compiled else 0.99), (n, cos)
    opt = torch.optim.AdamW(fused.parameters(), lr=3e-3)
    losses = []
    for _ in range(12):
        for p in fused.parameters():
            p.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = runner(idx, tgt)
            loss.backward()
        losses.append(loss.item())
        opt.step()
    assert losses[-1] < 0.85 * losses[0]
    assert ops.device_status() == 0
