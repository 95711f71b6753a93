"""Two-GPU check of the weight-gradient exchange through peer memory; skipped on a single-GPU box
(there the scattered GEMM and the slot sum are covered with one GPU standing in for every owner,
tests/test_gpu_gemm.py)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_scatter_matches_nccl_reduce_scatter():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(root, "tests", "peer_scatter_worker.py")]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
