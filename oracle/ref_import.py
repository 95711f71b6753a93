"""Import the reference's own quantization package on a CPU-only machine.

TEST INFRASTRUCTURE ONLY (used by tests/golden/make_golden.py and by CPU tests
that are skipped when the reference tree is absent).  No reference source is
copied: the modules are imported from where they lie (the `src` directory of a
reference checkout, named by the environment variable QUARTET_REF) after three shims:

1. TRITON_INTERPRET=1 so `mxfp4_forward_kernel` (mxfp4_triton.py:19-174) runs
   under Triton's numpy interpreter, and TORCHDYNAMO_DISABLE=1 so the
   `@torch.compile` on `QEQWtt_QEtQXttFn.backward` (backward.py:64) is inert.
2. A stand-in module `fast_hadamard_transform` whose `hadamard_transform(x, scale)`
   multiplies by the Sylvester matrix (the reference only uses it on an identity
   to build H, mxfp4.py:42-44), and a `torch.eye` wrapper that ignores
   `device="cuda"` (mxfp4.py:43 and import-time class bodies in quest.py /
   baselines.py ask for CUDA).
3. The autotuner object around the kernel (mxfp4_triton.py:8-17) needs a GPU to
   benchmark its configs; it is replaced by a launcher that always runs the
   interpreted kernel with BLOCK_SIZE = 16384 (the result does not depend on it).

The interpreter mis-handles bf16 tensors, so callers pass bf16-representable
fp32 tensors and an fp32 copy of the bf16-rounded rotation matrix.
"""
from __future__ import annotations

import os
import sys
import types

_REF = None


def load(ref_src: str | None = None):
    global _REF
    if _REF is not None:
        return _REF
    ref_src = ref_src or os.environ.get("QUARTET_REF")
    if not ref_src:
        raise FileNotFoundError("set QUARTET_REF to the `src` directory of a reference checkout")
    if not os.path.isdir(ref_src):
        raise FileNotFoundError(ref_src)
    os.environ["TRITON_INTERPRET"] = "1"
    os.environ["TORCHDYNAMO_DISABLE"] = "1"
    import torch

    from . import ref_math

    fht = types.ModuleType("fast_hadamard_transform")

    def hadamard_transform(x, scale=1.0):
        n = x.shape[-1]
        h = torch.ones(1, 1, dtype=torch.float64)
        while h.shape[0] < n:
            h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
        return (x.to(torch.float64) @ h * scale).to(x.dtype)

    fht.hadamard_transform = hadamard_transform
    sys.modules.setdefault("fast_hadamard_transform", fht)

    real_eye = torch.eye

    def eye_cpu(*a, **k):
        k.pop("device", None)
        return real_eye(*a, **k)

    torch.eye = eye_cpu
    if ref_src not in sys.path:
        sys.path.insert(0, ref_src)
    try:
        import models.quantization as mq
        import models.quantization.quantizers.mxfp4_triton as mt
    finally:
        torch.eye = real_eye

    tuner = mt.mxfp4_forward_kernel
    inner = tuner.fn  # the interpreted JIT function under the autotuner

    class _Launcher:
        def __getitem__(self, grid):
            def run(**kw):
                meta = {"BLOCK_SIZE": 16384}
                g = grid(meta) if callable(grid) else grid
                return inner[g](**kw, BLOCK_SIZE=16384)

            return run

    mt.mxfp4_forward_kernel = _Launcher()
    import contextlib

    @contextlib.contextmanager
    def cpu_eye():
        """Constructors of the reference quantizers ask torch.eye for device="cuda"."""
        torch.eye = eye_cpu
        try:
            yield
        finally:
            torch.eye = real_eye

    _REF = types.SimpleNamespace(mq=mq, mt=mt, ref_math=ref_math, torch=torch, cpu_eye=cpu_eye)
    return _REF
