"""The allocation-free entry point: same measurement as the workspace variant, with the per-SM cycle
counts in a device array inside the library.  It exists for callers that cannot allocate device memory
while they run (a frozen caching allocator, a plugin confined to buffers its host handed it, a hook that
runs on a nearly full device).  Named so that it is collected last."""
import ctypes as C

import pytest
import torch


def _lib():
    import __graft_entry__ as entry

    entry.build()
    from quartet_b200 import _lib

    return _lib.load()


def test_no_alloc_symbol_is_exported_and_rejects_bad_arguments_without_a_gpu():
    lib = _lib()
    fn = lib.quartet_probe_copy_ingress_noalloc
    out = C.c_double(0.0)
    assert fn(None, 1 << 20, 10, 2, 16384, 1, C.byref(out), None) != 0          # NULL source
    assert b"non-NULL" in lib.quartet_last_error_string()
    assert fn(C.c_void_p(256), 1 << 20, 10, 2, 16384, 9, C.byref(out), None) != 0  # more producers than supported
    assert fn(C.c_void_p(256), 1 << 20, 10, 32, 65536, 4, C.byref(out), None) != 0  # ring larger than shared memory


def test_probe_rejects_regions_and_sources_its_offsets_cannot_stay_inside():
    """Both probe variants: a region shorter than four chunks, a chunk that is not a multiple of 128 bytes
    and a source that is not 128-byte aligned are refused before anything is launched."""
    lib = _lib()
    out = C.c_double(0.0)
    for fn, extra in ((lib.quartet_probe_copy_ingress_noalloc, ()), (lib.quartet_probe_copy_ingress, (C.c_void_p(4096),))):
        def call(src, region, chunk):
            return fn(C.c_void_p(src), region, 10, 2, chunk, 1, *extra, C.byref(out), None)

        assert call(1024, 3 * 16384, 16384) == -4     # region < 4 chunks
        assert call(1024, 1 << 20, 16384 + 64) == -4  # chunk not a multiple of 128
        assert call(1024 + 16, 1 << 20, 16384) == -4  # source only 16-byte aligned
        assert b"128-byte aligned" in lib.quartet_last_error_string()


@pytest.mark.gpu
def test_no_alloc_variant_matches_workspace_variant_and_allocates_nothing():
    import __graft_entry__ as entry

    entry.build()
    from quartet_b200 import ops

    src = torch.ones(48 << 20, dtype=torch.uint8, device="cuda")
    ops.probe_copy_ingress_noalloc(src, iters=200)  # set-up call: symbol address, function attribute
    torch.cuda.synchronize()
    # two calls in a row through the C ABI, each against the workspace variant on the same arguments
    for _ in range(2):
        want = ops.probe_copy_ingress(region_mb=48, iters=2000, stages=6, chunk=16384, producers=2)
        torch.cuda.synchronize()
        free0, alloc0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
        got = ops.probe_copy_ingress_noalloc(src, iters=2000, stages=6, chunk=16384, producers=2)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0                      # nothing allocated on the device, by anyone
        assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
        assert 30.0 < got < 120.0                                        # bytes per clock per SM
        assert abs(got - want) / want < 0.15
    assert ops.device_status() == 0


@pytest.mark.gpu
def test_probe_on_a_region_of_a_few_chunks_stays_inside_it():
    """The smallest regions the validation admits (4 and 8 chunks, several producers): every copy must lie
    inside the region, so the run completes with a clean fault word and a plausible rate."""
    import __graft_entry__ as entry

    entry.build()
    from quartet_b200 import ops

    chunk = 16384
    guard = torch.zeros(16 * chunk, dtype=torch.uint8, device="cuda")  # the region is the first part of a larger buffer
    for n_chunks, producers in ((8, 2), (4, 4)):
        region = guard[: n_chunks * chunk]
        got = ops.probe_copy_ingress_noalloc(region, iters=500, stages=3, chunk=chunk, producers=producers)
        assert 10.0 < got < 200.0
    assert ops.device_status() == 0
