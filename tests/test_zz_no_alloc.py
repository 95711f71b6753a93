"""The allocation-free entry point: same measurement as the workspace variant, with the per-SM cycle
counts in a device array inside the library.  Named so that it is collected last."""
import ctypes as C

import pytest
import torch


def test_no_alloc_symbol_is_exported_and_rejects_bad_arguments_without_a_gpu():
    import __graft_entry__ as entry

    entry.build()
    from quartet_b200 import _lib

    lib = _lib.load()
    fn = lib.quartet_probe_copy_ingress_noalloc
    out = C.c_double(0.0)
    assert fn(None, 1 << 20, 10, 2, 16384, 1, C.byref(out), None) != 0          # NULL source
    assert b"non-NULL" in lib.quartet_last_error_string()
    assert fn(C.c_void_p(256), 1 << 20, 10, 2, 16384, 9, C.byref(out), None) != 0  # more producers than supported
    assert fn(C.c_void_p(256), 1 << 20, 10, 32, 65536, 4, C.byref(out), None) != 0  # ring larger than shared memory


@pytest.mark.gpu
def test_no_alloc_variant_matches_workspace_variant_and_allocates_nothing():
    import __graft_entry__ as entry

    entry.build()
    from quartet_b200 import ops

    src = torch.ones(48 << 20, dtype=torch.uint8, device="cuda")
    want = ops.probe_copy_ingress(region_mb=48, iters=2000, stages=6, chunk=16384, producers=2)
    ops.probe_copy_ingress_noalloc(src, iters=200)  # set-up call: symbol address, function attribute
    torch.cuda.synchronize()
    free0, alloc0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    got = ops.probe_copy_ingress_noalloc(src, iters=2000, stages=6, chunk=16384, producers=2)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0                      # nothing allocated on the device, by anyone
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
    assert 30.0 < got < 120.0                                        # bytes per clock per SM
    assert abs(got - want) / want < 0.15
    assert ops.device_status() == 0
