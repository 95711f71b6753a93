"""Builds the REFERENCE'S OWN model code (src/models/llama.py, unchanged, imported from a reference checkout
named by QUARTET_REF) on top of this package: `install()` registers quartet_b200.quantization as
`models.quantization`, the reference's argument parser supplies every default, and the flags are those of its
production launch script (main_setup.sh:78-127).  `tiktoken.get_encoding` (llama.py:182) needs the network
and is stubbed.  Nothing of the reference is copied; without a checkout the callers skip."""
import argparse
import contextlib
import importlib
import os
import sys
import types

PRODUCTION_FLAGS = [
    "--model", "llama", "--n-layer", "6", "--n-embd", "640", "--n-head", "5", "--vocab-size", "32000", "--sequence-length", "512",
    "--w-quant", "QuestMXFP4Quantizer", "--w-quant-kwargs", "{}", "--a-quant", "QuestMXFP4Quantizer", "--a-quant-kwargs", "{}",
    "--g-quant", "AlbertTsengQuantizer", "--g-quant-kwargs", '{"stochastic": true, "rerotate": "signs"}',
    "--backward-scheme", "Q(E)Q(Wt)t_Q(Et)Q(Xt)t", "--backward-scheme-kwargs", "{}",
]


def reference_src():
    ref = os.environ.get("QUARTET_REF")
    return ref if ref and os.path.isfile(os.path.join(ref, "models", "llama.py")) else None


@contextlib.contextmanager
def reference_on_this_package(extra_flags=()):
    """Yields (llama module, parsed args); restores sys.path / sys.modules afterwards."""
    import quartet_b200.quantization as Q

    ref = reference_src()
    names = ("models", "models.quantization", "models.quantization.quantizers", "models.quantization.backward", "models.llama",
             "models.base", "models.utils", "tiktoken", "config", "config.base", "distributed", "distributed.backend",
             "distributed.ddp", "distributed.single")
    saved = {k: sys.modules.get(k) for k in names}
    sys.path.insert(0, ref)
    try:
        for k in names:
            sys.modules.pop(k, None)
        tk = types.ModuleType("tiktoken")
        tk.get_encoding = lambda name: types.SimpleNamespace(n_vocab=50257)
        sys.modules["tiktoken"] = tk
        pkg = types.ModuleType("models")
        pkg.__path__ = [os.path.join(ref, "models")]
        sys.modules["models"] = pkg
        Q.install("models.quantization")
        config = importlib.import_module("config")
        args = config.parse_args_with_format("base", argparse.ArgumentParser(), PRODUCTION_FLAGS + list(extra_flags), None)
        llama = importlib.import_module("models.llama")
        yield llama, args
    finally:
        sys.path.remove(ref)
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
