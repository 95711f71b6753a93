"""quartet_b200: the MXFP4 quantized-linear hot path of Quartet, hand-written for B200 (sm_100a).

The compute lives in libquartet_b200.so behind a C ABI (include/quartet_b200.h); this package is the
host-side mirror of the reference's `models.quantization` interface on top of it.
"""
from . import ops  # noqa: F401
