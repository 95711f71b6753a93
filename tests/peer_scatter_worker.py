"""One rank of the two-GPU check of the peer-memory weight-gradient exchange (started by
tests/test_gpu_peer_scatter.py, one process per GPU): the same layer runs a step with the NCCL
reduce-scatter of full partials and a step with the GEMM storing rows straight to their owner, from
identical seeds, and the owned shards must agree."""
import os
import random
import sys

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from quartet_b200 import ops
    from quartet_b200.quantization import BACKWARD_SCHEMES, QUANTIZER_CLASSES, QuantizedLinear
    from quartet_b200.shard import PeerWgradScatter, WgradReduceScatter

    k, n, tokens = 512, 1024, 512
    torch.manual_seed(5)
    lin = QuantizedLinear(
        k, n, bias=False,
        weight_quantizer=QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
        activation_quantizer=QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
        gradient_quantizer=QUANTIZER_CLASSES["AlbertTsengQuantizer"](stochastic=True, rerotate="signs"),
        backward_scheme=BACKWARD_SCHEMES["Q(E)Q(Wt)t_Q(Et)Q(Xt)t"](),
    ).cuda()
    g = torch.Generator().manual_seed(100 + rank)  # every rank its own token rows
    x = torch.randn(tokens, k, generator=g).to(torch.bfloat16).cuda().requires_grad_(True)
    e = (torch.randn(tokens, n, generator=g) * 1e-2).to(torch.bfloat16).cuda()

    def run(sink):
        lin.wgrad_sink = sink
        lin.weight.grad = None
        random.seed(7), torch.manual_seed(7)  # same rounding seeds and rotation signs in both runs
        lin(x).backward(e)

    reducer = WgradReduceScatter(world)
    for transport in ("store", "copy"):  # rows stored by the GEMM epilogue / pushed by the DMA engines
        sink = PeerWgradScatter(transport=transport)
        shards = []
        for step in range(3):  # three steps: both receive buffers of the layer get reused
            run(None)
            reducer.submit(lin.weight.grad)
            want = reducer.wait()[0]
            run(sink)
            assert lin.weight.grad is None
            got = sink.wait()[0]
            assert got is lin.weight.grad_shard
            torch.cuda.synchronize()
            err = ((got - want).abs().max() / want.abs().max()).item()
            assert err < 1e-6, (transport, step, err)  # same addends, different summation order
            shards.append(got.clone())
        assert torch.equal(shards[0], shards[1]) and torch.equal(shards[1], shards[2])  # deterministic
        assert ops.device_status() == 0
        sink.close()
    dist.destroy_process_group()
    print(f"rank {rank} ok", flush=True)


if __name__ == "__main__":
    main()
