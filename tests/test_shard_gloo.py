"""Row sharding and the wgrad exchange on two CPU ranks (gloo)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from quartet_b200.shard import shard_rows


def test_shard_rows_cover_and_align():
    for total, world in ((16384, 8), (1280, 3), (128, 1), (640, 4), (256, 8)):
        spans = [shard_rows(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c
        assert all(lo % 128 == 0 and hi % 128 == 0 for lo, hi in spans)
    with pytest.raises(ValueError):
        shard_rows(100, 2, 0)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import ref_math as rm
    from quartet_b200.shard import WgradReduceScatter

    gen = torch.Generator().manual_seed(0)
    m, k, n = 256, 64, 96
    x = torch.randn(m, k, generator=gen)
    e = torch.randn(m, n, generator=gen)
    lo, hi = shard_rows(m, world, rank)
    # the partial wgrad of this rank's token rows; groups of 32 tokens never straddle ranks
    dw_part = e[lo:hi].T @ x[lo:hi]
    red = WgradReduceScatter(world)
    red.submit(dw_part)
    red.submit(2 * dw_part)
    a, b = red.wait()
    full = (e.T @ x) / world
    rows = n // world
    ok = torch.allclose(a, full[rank * rows:(rank + 1) * rows], atol=1e-4) and torch.allclose(b, 2 * a, atol=1e-4)
    # the peer-memory exchange in host arithmetic: slot r of this owner's receive buffer holds the owner's row range of
    # rank r's partial; the slots are added in rank order and scaled by 1/world -- the same shard as above
    parts = [torch.empty_like(dw_part) for _ in range(world)]
    dist.all_gather(parts, dw_part)
    slots = torch.stack([part_r[rank * rows:(rank + 1) * rows] for part_r in parts])
    acc = slots[0].clone()
    for r in range(1, world):
        acc = acc + slots[r]
    ok = ok and torch.allclose(acc * (1.0 / world), a, atol=1e-4)
    # ... and the GPU implementation refuses a host backend instead of falling back to something else
    from quartet_b200.shard import PeerWgradScatter

    try:
        PeerWgradScatter()
        ok = False
    except RuntimeError:
        pass
    # per-rank quantization of the transposed operand equals the single-process result group for group
    h = rm.hadamard32()
    u = torch.rand(n, m, generator=gen)
    whole = rm.quant_bwd(e.T.contiguous(), h, u)
    part = rm.quant_bwd(e[lo:hi].T.contiguous(), h, u[:, lo:hi].contiguous())
    ok = ok and bool((part.codes == whole.codes[:, lo:hi]).all()) and bool((part.e8m0 == whole.e8m0[:, lo // 32:hi // 32]).all())
    q.put((rank, ok))
    dist.destroy_process_group()


def test_two_rank_wgrad_exchange():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]
