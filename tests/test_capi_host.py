"""Host-side checks that need no GPU: the shared object loads, exports every symbol the header
declares, and rejects bad arguments with error codes before touching a device."""
import ctypes as C
import os
import re

import pytest

import __graft_entry__ as entry
from quartet_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    entry.build()
    return _lib.load()


def test_header_symbols_are_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "quartet_b200.h")).read()
    declared = set(re.findall(r"\b(quartet_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"
    for name in declared:
        assert hasattr(lib, name), f"{name} not exported"
    assert lib.quartet_version() >= 100


def test_sf_layout_helpers_match_oracle(lib):
    from oracle import ref_math as rm

    for r, k, pk in ((0, 0, 4), (31, 3, 4), (32, 0, 8), (127, 7, 8), (128, 4, 12), (1000, 37, 40)):
        assert lib.quartet_sf_offset(r, k, pk) == rm.sf_offset(r, k, pk)
    assert lib.quartet_sf_bytes(200, 320) == 256 * 12
    assert lib.quartet_sf_bytes(128, 128) == 512


def test_rejections(lib):
    buf = (C.c_uint8 * 4096)()
    p = C.cast(buf, C.c_void_p)
    # NULL pointers
    assert lib.quartet_quant_fwd(None, 0, 128, 128, 0.17, 0.5, p, p, None, None) == -1
    assert b"non-NULL" in lib.quartet_last_error_string()
    # bad extents
    assert lib.quartet_quant_fwd(p, 0, 128, 96, 0.17, 0.5, p, p, None, None) == -2
    assert lib.quartet_quant_fwd(p, 0, 0, 128, 0.17, 0.5, p, p, None, None) == -2
    assert lib.quartet_quant_bwd_t(p, 0, 100, 128, 0.17, 0, None, 1, 0, 0, None, p, p, None) == -2
    assert lib.quartet_gemm_mxfp4_tn(p, p, p, p, 128, 128, 64, 1.0, None, 0.17, p, 0, None) == -2
    # bad enums
    assert lib.quartet_quant_fwd(p, 7, 128, 128, 0.17, 0.5, p, p, None, None) == -4
    assert lib.quartet_quant_group32(p, 0, 128, 128, 2, 0.5, 0, 0, 0, None, p, p, None, None) == -4   # kind
    assert lib.quartet_quant_group32(p, 0, 128, 128, 1, 0.5, 2, 0, 0, None, p, p, None, None) == -1   # noise mode without a noise tensor
    assert lib.quartet_quant_group32(p, 0, 128, 100, 0, 0.5, 0, 0, 0, None, p, p, None, None) == -2
    # misaligned pointer
    q = C.c_void_p(p.value + 4)
    assert lib.quartet_dequant(q, p, 1, 32, 1.0, p, 1, None) == -3
    with pytest.raises(ValueError):
        _lib.check(-2, "x")


def test_host_stager_has_no_cpu_path():
    import torch

    from quartet_b200.staging import HostStager

    with pytest.raises(RuntimeError):
        HostStager(torch.device("cpu"))
