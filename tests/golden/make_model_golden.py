"""Generate tests/golden/llama_tiny_step.npz: one training step of the REFERENCE'S OWN model code on the
reference's own quantization package, on CPU.

    QUARTET_REF=<reference checkout>/src python tests/golden/make_model_golden.py

The reference's `Llama` (src/models/llama.py, unchanged, built through the reference's argument parser) runs
forward + backward in fp32 with its Triton kernel under the interpreter (oracle/ref_import.py).  Configuration:
2 blocks, width 128, 1 head, SwiGLU hidden 512, vocabulary 256, 2 x 128 tokens; quantizers and scheme as in
main_setup.sh:78-93 except that the gradient quantizer rounds to nearest and keeps its rotation
(`{"stochastic": false}`), so that the step is deterministic and comparable bit-pattern-free.  All parameters
are rounded to bf16-representable values and stored as 16-bit patterns; stored outputs: the loss, a sample of
the logits, and per parameter the gradient's norm and its first row.
"""
from __future__ import annotations

import argparse
import importlib
import os
import sys
import types

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref_import  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "llama_tiny_step.npz")
FLAGS = [
    "--model", "llama", "--n-layer", "2", "--n-embd", "128", "--n-head", "1", "--vocab-size", "256", "--sequence-length", "128",
    "--multiple-of", "256",
    "--w-quant", "QuestMXFP4Quantizer", "--w-quant-kwargs", "{}", "--a-quant", "QuestMXFP4Quantizer", "--a-quant-kwargs", "{}",
    "--g-quant", "AlbertTsengQuantizer", "--g-quant-kwargs", '{"stochastic": false}',
    "--backward-scheme", "Q(E)Q(Wt)t_Q(Et)Q(Xt)t", "--backward-scheme-kwargs", "{}",
]


def main():
    ref = ref_import.load()  # the reference's models.quantization, interpreted kernel, CPU shims
    import torch

    tk = types.ModuleType("tiktoken")
    tk.get_encoding = lambda name: types.SimpleNamespace(n_vocab=50257)
    sys.modules["tiktoken"] = tk
    config = importlib.import_module("config")
    args = config.parse_args_with_format("base", argparse.ArgumentParser(), FLAGS, None)
    llama = importlib.import_module("models.llama")
    torch.manual_seed(0)
    with ref.cpu_eye():
        model = llama.Llama(args)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(p.to(torch.bfloat16).to(torch.float32))
    gen = torch.Generator().manual_seed(1)
    idx = torch.randint(0, 256, (2, 128), generator=gen)
    tgt = torch.randint(0, 256, (2, 128), generator=gen)
    out = model(idx, targets=tgt, get_logits=True)
    out["loss"].backward()
    blob = {"idx": idx.numpy(), "targets": tgt.numpy(), "loss": np.float32(out["loss"].item()),
            "logits_sample": out["logits"][:, ::8, :].detach().numpy(), "rmsnorm_eps": np.float32(args.rmsnorm_eps)}
    for name, p in model.named_parameters():
        blob["param:" + name] = p.detach().to(torch.bfloat16).view(torch.int16).numpy()
        g = p.grad.detach()
        blob["gnorm:" + name] = np.float32(g.norm().item())
        blob["grow:" + name] = g.reshape(g.shape[0], -1)[0].numpy() if g.dim() > 1 else g.numpy()
    np.savez_compressed(OUT, **blob)
    print("loss", out["loss"].item(), "parameters", sum(p.numel() for p in model.parameters()), "->", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
