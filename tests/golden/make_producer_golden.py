"""Generate tests/golden/producer_steps.npz: the two elementwise steps that feed a quantized layer, computed by
the REFERENCE'S OWN model code on CPU.

    QUARTET_REF=<reference checkout>/src python tests/golden/make_producer_golden.py

* RMSNorm: the reference's `RMSNorm` module (src/models/llama.py:64-75) with a non-trivial weight, on fp32 rows and
  on bf16 rows (the bf16 case exercises `.type_as(x)`: the normalised value is rounded before the fp32 weight
  multiplies it, and the result is fp32).
* SwiGLU: the reference's `LlamaMLP.forward` (llama.py:112-114) with both of its linears replaced by identities,
  so that it returns `silu(up) * gate` of its input; fp32 and bf16.
bf16 tensors are stored as their 16-bit patterns.  tests/test_oracle_golden.py holds oracle.ref_math.rmsnorm /
swiglu to these outputs bit for bit.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref_import  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "producer_steps.npz")


def bits(t):
    import torch

    return t.view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def main():
    ref_import.load()
    import torch

    tk = types.ModuleType("tiktoken")
    tk.get_encoding = lambda name: types.SimpleNamespace(n_vocab=50257)
    sys.modules["tiktoken"] = tk
    llama = importlib.import_module("models.llama")
    gen = torch.Generator().manual_seed(4)
    blob = {}
    eps = 1e-5
    norm = llama.RMSNorm(256, eps=eps)
    with torch.no_grad():
        norm.weight.copy_(1.0 + 0.1 * torch.randn(256, generator=gen))
    x = torch.randn(48, 256, generator=gen) * torch.logspace(-2, 2, 48).reshape(-1, 1)
    x[5] = 0.0
    blob["rms_eps"], blob["rms_weight"] = np.float32(eps), norm.weight.detach().numpy()
    for name, xin in (("f32", x), ("bf16", x.to(torch.bfloat16))):
        with torch.no_grad():
            out = norm(xin)
        assert out.dtype == torch.float32
        blob[f"rms_x_{name}"], blob[f"rms_out_{name}"] = bits(xin), out.numpy()
    mlp = llama.LlamaMLP.__new__(llama.LlamaMLP)
    torch.nn.Module.__init__(mlp)
    mlp.hidden_dim, mlp.w12, mlp.c_proj = 192, torch.nn.Identity(), torch.nn.Identity()
    h = 3.0 * torch.randn(40, 384, generator=gen)
    h[0, :64] = torch.linspace(-40, 40, 64)
    for name, hin in (("f32", h), ("bf16", h.to(torch.bfloat16))):
        with torch.no_grad():
            out = mlp(hin)
        assert out.dtype == hin.dtype and out.shape == (40, 192)
        blob[f"swiglu_h_{name}"], blob[f"swiglu_out_{name}"] = bits(hin), bits(out)
    np.savez_compressed(OUT, **blob)
    print("->", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
