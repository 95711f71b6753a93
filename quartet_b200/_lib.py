"""ctypes binding of libquartet_b200.so (the C ABI declared in include/quartet_b200.h).

There is no fallback: if the shared object is missing or a call is rejected, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# QUARTET_B200_LIB points at an alternative build of the same library (e.g. one compiled with tracing)
LIB_PATH = os.environ.get("QUARTET_B200_LIB") or os.path.join(_PKG, "lib", "libquartet_b200.so")

_p, _i, _i64, _u32, _u64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_uint32, C.c_uint64, C.c_float

# name -> (restype, argtypes); mirrors include/quartet_b200.h one to one
SIGNATURES = {
    "quartet_quant_fwd": (_i, [_p, _i, _i64, _i64, _f, _f, _p, _p, _p, _p]),
    "quartet_rms_stats": (_i, [_p, _i, _i64, _i64, _f, _p, _p]),
    "quartet_quant_fwd_rmsnorm": (_i, [_p, _i, _i64, _i64, _p, _f, _p, _f, _f, _p, _p, _p, _p]),
    "quartet_quant_fwd_swiglu": (_i, [_p, _i, _i64, _i64, _f, _f, _p, _p, _p, _p]),
    "quartet_swiglu": (_i, [_p, _i, _i64, _i64, _p, _p]),
    "quartet_quant_bwd": (_i, [_p, _i, _i64, _i64, _f, _u32, _p, _i, _u64, _u64, _p, _p, _p, _p]),
    "quartet_quant_group32": (_i, [_p, _i, _i64, _i64, _i, _f, _i, _u64, _u64, _p, _p, _p, _p, _p]),
    "quartet_quant_bwd_t": (_i, [_p, _i, _i64, _i64, _f, _u32, _p, _i, _u64, _u64, _p, _p, _p, _p]),
    "quartet_quant_bwd_dual": (_i, [_p, _i, _i64, _i64, _f, _u32, _p, _i, _u64, _u64, _u64, _p, _p, _p, _p, _p]),
    "quartet_requant_t": (_i, [_p, _p, _i64, _i64, _f, _f, _u32, _p, _i, _u64, _u64, _p, _p, _p, _p]),
    "quartet_gemm_mxfp4_tn": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _f, _p, _f, _p, _i, _p]),
    "quartet_gemm_mxfp4_tn_scatter": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _f, _p, _f, _p, C.c_int32, _i64, _p]),
    "quartet_shard_reduce": (_i, [_p, C.c_int32, _i64, _f, _p, _p]),
    "quartet_peer_alloc": (_i, [_u64, C.POINTER(C.c_void_p), _p]),
    "quartet_peer_free": (_i, [_p]),
    "quartet_peer_open": (_i, [_p, C.POINTER(C.c_void_p)]),
    "quartet_peer_close": (_i, [_p]),
    "quartet_peer_copy": (_i, [_p, _p, _u64, _p]),
    "quartet_probe_copy_ingress": (_i, [_p, _u64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _p, C.POINTER(C.c_double), _p]),
    "quartet_probe_copy_ingress_noalloc": (_i, [_p, _u64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_double), _p]),
    "quartet_fold_signs": (_i, [_p, _i, _p, _p]),
    "quartet_selftest_wait_timeout": (_i, [_p, _p]),
    "quartet_linear_fwd": (_i, [_p, _i, _p, _i, _i64, _i64, _i64, _f, _f, _f, _p, _p, _p, _p, _p, _p, _p, _i, _p]),
    "quartet_linear_bwd_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "quartet_linear_bwd": (_i, [_p, _i, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _f, _u32, _p, _i, C.POINTER(C.c_uint64), _u64, _f, _f, _f, _p,
                                _p, _i, _p, _i, _p]),
    "quartet_unrotate_mask": (_i, [_p, _i, _p, _i64, _i64, _f, _p, _i, _p]),
    "quartet_dequant": (_i, [_p, _p, _i64, _i64, _f, _p, _i, _p]),
    "quartet_sf_offset": (_i64, [_i64, _i64, _i64]),
    "quartet_sf_bytes": (_i64, [_i64, _i64]),
    "quartet_device_status": (_i, [C.POINTER(C.c_int32)]),
    "quartet_last_error_string": (C.c_char_p, []),
    "quartet_version": (_i, []),
}

_lib = None


class QuartetError(RuntimeError):
    pass


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise QuartetError(
            f"{LIB_PATH} is missing: build it with `python -m quartet_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc != 0:
        msg = load().quartet_last_error_string().decode()
        exc = ValueError if rc in (-1, -2, -3, -4) else QuartetError
        raise exc(f"{what} failed ({rc}): {msg}")
