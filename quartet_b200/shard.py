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


class PeerSetupError(RuntimeError):
    """Raised on EVERY rank when any rank failed to allocate or map the receive buffers."""


class PeerWgradScatter:
    """The weight-gradient exchange folded into the wgrad GEMM.

    Rank r's GEMM stores the rows of its partial dW that rank o owns directly into slot r of a
    receive buffer in o's memory (TMA stores over NVLink while the tiles are computed,
    `ops.gemm_mxfp4_tn_scatter`); a one-element all-reduce on a side stream then orders "every rank's
    GEMM has finished" before the owner sums its slots (`ops.shard_reduce`, fixed order, scaled by
    1/world as the reference's DDP averages, src/distributed/ddp.py:43).  No gradient bytes go through a
    library collective and no full-size partial is ever written to local memory.

    Attach with `layer.wgrad_sink = sink`; the layer's backward then returns no dense weight gradient
    and the averaged shard (rows [rank*N/world, (rank+1)*N/world)) is found in `layer.weight.grad_shard`
    after `sink.wait()`.  Call `wait()` at least once per step: the two receive buffers of a layer alternate
    from use to use, and a buffer is reused only after the sum of its previous contents has been issued.
    """

    MAX_WORLD = 8

    def __init__(self, group=None, device=None, transport: str = "store"):
        from . import ops

        if transport not in ("store", "copy"):
            raise ValueError("transport is 'store' (GEMM epilogue stores to peers) or 'copy' (DMA engines push local rows)")
        self.transport = transport
        self.ops = ops
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if dist.get_backend(group) != "nccl":
            raise RuntimeError("PeerWgradScatter moves gradients through GPU peer memory; it needs the nccl backend")
        if self.world > self.MAX_WORLD:
            raise ValueError(f"at most {self.MAX_WORLD} ranks (one NVLink domain)")
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.stream = torch.cuda.Stream(device=self.device)
        self.copy_streams = [torch.cuda.Stream(device=self.device) for _ in range(4)]
        self.flag = torch.zeros(1, device=self.device)
        self.plans = {}
        self.pending = []
        self.unreduced = []   # exchanges in flight: (weight, plan, parity, event "all ranks' rows have landed")
        self.lag = 1          # how many exchanges may stay in flight before the compute stream is made to wait for the oldest

    def accepts(self, rows: int, cols: int, dtype: torch.dtype) -> bool:
        return (dtype == torch.float32 and rows % 256 == 0 and cols % 256 == 0 and rows % self.world == 0
                and (rows // self.world) % 32 == 0)

    def prepare(self, weight: torch.Tensor):
        """Collective: allocates this layer's receive buffers and maps every peer's.  All ranks must
        prepare their layers in the same order."""
        key = id(weight)
        if key in self.plans:
            return self.plans[key]
        rows, cols = weight.shape
        if not self.accepts(rows, cols, weight.dtype):
            raise ValueError(f"weight [{rows}, {cols}] {weight.dtype} cannot be scattered over {self.world} ranks")
        rpo = rows // self.world
        slot_bytes = rpo * cols * 4
        # Every rank walks through the same collectives whatever fails locally, and all ranks agree on
        # the outcome before anyone raises: a rank that cannot allocate or map must not leave the others
        # waiting in a collective.
        mine, handles, opened, error = [], [], [], None
        try:
            for _ in range(2):
                ptr, h = self.ops.peer_alloc(self.world * slot_bytes, self.device)
                mine.append(ptr), handles.append(h)
        except Exception as exc:  # noqa: BLE001 - reported after the agreement below
            error = exc
        gathered = [None] * self.world
        dist.all_gather_object(gathered, handles if error is None else None, group=self.group)
        dst = []
        if error is None and all(g is not None for g in gathered):
            try:
                for parity in range(2):
                    bases = []
                    for o in range(self.world):
                        if o == self.rank:
                            bases.append(mine[parity])
                        else:
                            p = self.ops.peer_open(gathered[o][parity], self.device)
                            opened.append(p)
                            bases.append(p)
                    dst.append([b + self.rank * slot_bytes for b in bases])
            except Exception as exc:  # noqa: BLE001
                error = exc
        elif error is None:
            error = RuntimeError("another rank could not allocate its receive buffers")
        ok = torch.tensor([0.0 if error is not None else 1.0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if ok.item() < 1.0:
            for p in opened:
                self.ops.peer_close(p, self.device)
            dist.barrier(group=self.group)  # nobody frees a buffer a peer still has mapped
            for p in mine:
                self.ops.peer_free(p, self.device)
            raise PeerSetupError(f"peer receive buffers could not be set up on every rank: {error or 'failure on another rank'}")
        plan = {"rows": rows, "cols": cols, "rpo": rpo, "mine": mine, "dst": dst, "opened": opened, "uses": 0}
        self.plans[key] = plan
        return plan

    def wgrad(self, weight, a, a_sf, b, b_sf, alpha, mask, had_scale):
        plan = self.prepare(weight)
        # Exchanges of earlier layers have usually completed by now: sum their slots at full speed.  An exchange of
        # THIS layer still in flight is joined first: a receive buffer is reused only after the sum of its previous
        # contents has been issued on every rank (that sum precedes this layer's next completion signal).
        self._reduce_ready(block=any(pl is plan for _, pl, _, _ in self.unreduced))
        parity = plan["uses"] & 1
        plan["uses"] += 1
        dense = None
        main = torch.cuda.current_stream(self.device)
        if self.transport == "store":
            self.ops.gemm_mxfp4_tn_scatter(a, a_sf, b, b_sf, plan["dst"][parity], plan["rpo"], alpha, mask=mask, had_scale=had_scale)
        else:
            dense = self.ops.gemm_mxfp4_tn(a, a_sf, b, b_sf, alpha, mask=mask, had_scale=had_scale, out_dtype=torch.float32)
        produced = torch.cuda.Event()
        produced.record(main)
        if dense is not None:
            # the DMA engines push each owner's rows while the compute stream moves on, several copies at a time
            # (one stream per copy engine in use); peers are visited starting after this rank so that no two ranks
            # target one GPU at the same time
            slot_bytes = plan["rpo"] * plan["cols"] * 4
            for step in range(self.world):
                o = (self.rank + 1 + step) % self.world
                cs = self.copy_streams[step % len(self.copy_streams)]
                cs.wait_event(produced)
                with torch.cuda.stream(cs):
                    self.ops.peer_copy(plan["dst"][parity][o], dense.data_ptr() + o * slot_bytes, slot_bytes, self.device)
                dense.record_stream(cs)
            for cs in self.copy_streams:
                self.stream.wait_stream(cs)
        else:
            self.stream.wait_event(produced)
        with torch.cuda.stream(self.stream):
            dist.all_reduce(self.flag, group=self.group)  # every rank's rows of this layer have landed everywhere
            arrived = torch.cuda.Event()
            arrived.record(self.stream)
        # The slot sum runs on the COMPUTE stream, after `arrived`, when a later layer's backward (or wait()) comes
        # by: on a side stream it would run beside the persistent GEMM, get a handful of SMs and delay the CTAs of
        # the next GEMM launch that need them.
        self.unreduced.append((weight, plan, parity, arrived))
        return None

    def _reduce_ready(self, block: bool = False):
        """Sums the slots of exchanges that have completed (all of them if `block`), oldest first, on the compute stream."""
        main = torch.cuda.current_stream(self.device)
        while self.unreduced:
            weight, plan, parity, arrived = self.unreduced[0]
            if not block and len(self.unreduced) <= self.lag and not arrived.query():
                break
            self.unreduced.pop(0)
            main.wait_event(arrived)
            out = torch.empty(plan["rpo"], plan["cols"], dtype=torch.float32, device=self.device)
            self.ops.shard_reduce(plan["mine"][parity], self.world, plan["rpo"] * plan["cols"], 1.0 / self.world, out)
            weight.grad_shard = out
            self.pending.append(out)

    def wait(self):
        """Joins every exchange submitted so far; returns the owned, averaged shards in submission order."""
        self._reduce_ready(block=True)
        self.ops.raise_on_fault("weight-gradient exchange")  # only with QUARTET_CHECK_FAULTS=1
        out, self.pending = self.pending, []
        return out

    def close(self):
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for plan in self.plans.values():
            for p in plan["opened"]:
                self.ops.peer_close(p, self.device)
        dist.barrier(group=self.group)
        for plan in self.plans.values():
            for p in plan["mine"]:
                self.ops.peer_free(p, self.device)
        self.plans = {}
