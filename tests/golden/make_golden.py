"""Generate tests/golden/*.npz by running the reference's own code on CPU.

Run from the repo root in a container that has the reference tree:

    QUARTET_REF=<reference checkout>/src python tests/golden/make_golden.py

The reference kernel (src/models/quantization/quantizers/mxfp4_triton.py) is
executed under the Triton interpreter through oracle/ref_import.py; the
reference QuantizedLinear (src/models/quantization/__init__.py) is run forward
and backward with the production quantizer/scheme names of main_setup.sh:78-92.
Inputs are bf16-representable fp32 (the interpreter cannot take bf16).
"""
from __future__ import annotations

import os
import random
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref_import  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def bf16_round(t):
    import torch

    return t.to(torch.bfloat16).to(torch.float32)


def student_t_outliers(rows, cols, seed):
    """Quantize-sweep value distribution: Student-t(3), 1 % of channels x 20."""
    import torch

    rng = np.random.default_rng(seed)
    x = rng.standard_t(3, (rows, cols)).astype(np.float32)
    ch = rng.choice(cols, max(1, round(0.01 * cols)), replace=False)
    x[:, ch] *= 20
    return bf16_round(torch.from_numpy(x))


def main():
    ref = ref_import.load()
    import torch

    rm = ref.ref_math
    wrapper = ref.mt.mxfp4_forward_kernel_wrapper
    h = rm.hadamard32(torch.bfloat16)

    # ---- 1. the quantizer kernel, three branches, two value distributions ----
    gen = torch.Generator().manual_seed(0)
    cases = {
        "gauss": bf16_round(torch.randn(96, 256, generator=gen)),
        "grad": bf16_round(torch.randn(96, 256, generator=gen) * 1e-3),
        "student": student_t_outliers(64, 512, 0),
    }
    # edge rows: an all-zero group, a single spike, a constant run, tiny values
    edge = torch.zeros(8, 128)
    edge[1, 5] = 3.0
    edge[2, 32:64] = 0.5
    edge[3, :] = 1e-30
    edge[4, :] = bf16_round(torch.randn(128, generator=gen) * 1e4)
    edge[5, 64:96] = bf16_round(torch.randn(32, generator=gen))
    cases["edge"] = bf16_round(edge)
    signs = int(torch.randint(0, 2, (32,), generator=gen).mul(2 ** torch.arange(32)).sum().item()) & 0xFFFFFFFF
    h_b = h * rm.signs_to_diag(signs)[None, :]
    blob = {"signs": np.uint32(signs)}
    for name, x in cases.items():
        out_q, mask_q = wrapper(x, h, return_clip_mask=True, stochastic_round=False, quest=True,
                                gaussian_scale=2.92247856 / 6.0)
        random.seed(1234)
        seed = random.randint(0, 1000000)
        random.seed(1234)
        out_sr, _ = wrapper(x, h_b, return_clip_mask=False, stochastic_round=True, quest=False, gaussian_scale=3 / 4)
        out_rtn, _ = wrapper(x, h_b, return_clip_mask=False, stochastic_round=False, quest=False, gaussian_scale=3 / 4)
        blob[f"{name}_x"] = x.numpy()
        blob[f"{name}_quest_out"] = out_q.numpy()
        blob[f"{name}_quest_mask"] = mask_q.numpy()
        blob[f"{name}_sr_seed"] = np.int64(seed)
        blob[f"{name}_sr_out"] = out_sr.numpy()
        blob[f"{name}_absmax_rtn_out"] = out_rtn.numpy()
    np.savez_compressed(os.path.join(OUT, "quantizer_kernel.npz"), **blob)

    # ---- 2. one QuantizedLinear, forward + backward, production configuration ----
    mq = ref.mq
    m, k, n = 128, 128, 256
    torch.manual_seed(0)
    random.seed(0)
    with ref.cpu_eye():
        lin = mq.QuantizedLinear(
            k, n, bias=False,
            weight_quantizer=mq.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
            activation_quantizer=mq.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
            gradient_quantizer=mq.QUANTIZER_CLASSES["AlbertTsengQuantizer"](stochastic=True, rerotate="signs"),
            backward_scheme=mq.BACKWARD_SCHEMES["Q(E)Q(Wt)t_Q(Et)Q(Xt)t"](),
        )
    for q in (lin.weight_quantizer, lin.activation_quantizer, lin.backward_scheme.g_quantizer):
        q.hadamard_matrix = h.clone()
    with torch.no_grad():
        lin.weight.copy_(bf16_round(torch.randn(n, k, generator=gen) * 0.02))
    x = bf16_round(torch.randn(m, k, generator=gen)).requires_grad_(True)
    e = bf16_round(torch.randn(m, n, generator=gen) * 1e-3)
    y = lin(x)
    # the four stochastic-rounding seeds the wrapper will draw, in call order (mxfp4_triton.py:196-197)
    state = random.getstate()
    seeds = [random.randint(0, 1000000) for _ in range(4)]
    random.setstate(state)
    y.backward(e)
    h_after = lin.backward_scheme.g_quantizer.hadamard_matrix
    sign_vec = (h_after[0] / h[0]).round()  # row 0 of H is all +, so this is diag(s)
    sign_word = int(sum((1 << j) for j in range(32) if sign_vec[j] < 0))
    np.savez_compressed(
        os.path.join(OUT, "linear_fwd_bwd.npz"),
        x=x.detach().numpy(), w=lin.weight.detach().numpy(), e=e.numpy(),
        y=y.detach().numpy(), dx=x.grad.numpy(), dw=lin.weight.grad.numpy(),
        seeds=np.array(seeds, dtype=np.int64), signs=np.uint32(sign_word),
    )
    print("wrote", os.listdir(OUT))


if __name__ == "__main__":
    main()
