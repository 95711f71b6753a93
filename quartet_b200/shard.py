"""Multi-GPU plumbing of the path: one process per GPU, token rows sharded, no collective for
quantize / forward / dgrad, and one exchange step -- the weight-gradient partials.

Every rank holds rows [lo, hi) of X and E (a multiple of 128 rows, so each 32-token scale group of
the wgrad operands lives on exactly one rank) and computes a partial dW over its own tokens; the
partials are averaged across ranks (the reference's DDP averages gradients, src/distributed/ddp.py:43)
with a reduce-scatter, so each rank ends up owning rows [r*N/G, (r+1)*N/G) of the averaged dW.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(total_rows: int, world: int, rank: int, multiple: int = 128):
    """Contiguous, `multiple`-aligned split of `total_rows` over `world` ranks: (lo, hi) of `rank`.
    Earlier ranks take the remainder blocks, so sizes differ by at most one block."""
    if total_rows % multiple != 0:
        raise ValueError(f"{total_rows} rows is not a multiple of {multiple}")
    blocks = total_rows // multiple
    base, extra = divmod(blocks, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * multiple, hi * multiple


class WgradReduceScatter:
    """Averages weight-gradient partials across ranks on a side stream so that the exchange of one
    layer overlaps the backward of the next.  submit() returns immediately; wait() joins and
    returns the owned shards in submission order."""

    def __init__(self, world: int | None = None, group=None):
        self.group = group
        self.world = world or dist.get_world_size(group)
        self.backend = dist.get_backend(group)
        self.cuda = self.backend == "nccl"
        self.stream = torch.cuda.Stream() if self.cuda else None
        self.pending = []

    def submit(self, dw: torch.Tensor):
        n = dw.shape[0]
        if n % self.world != 0:
            raise ValueError(f"{n} output rows do not split over {self.world} ranks")
        if self.cuda:
            out = torch.empty(n // self.world, *dw.shape[1:], dtype=dw.dtype, device=dw.device)
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                dist.reduce_scatter_tensor(out, dw, op=dist.ReduceOp.AVG, group=self.group)
            dw.record_stream(self.stream)
            self.pending.append(out)
        else:
            # host backends (used by the CPU tests of this bookkeeping) have no reduce-scatter
            buf = dw.clone()
            dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group)
            r = dist.get_rank(self.group)
            rows = n // self.world
            self.pending.append(buf[r * rows:(r + 1) * rows] / self.world)

    def wait(self):
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.stream)
        out, self.pending = self.pending, []
        return out
