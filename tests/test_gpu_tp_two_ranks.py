"""Two ranks on two GPUs: the tensor-parallel block linears with the all-reduce fused into the row-parallel GEMM, and with
the library's one-shot all-reduce kernel over peer memory, give,
bit for bit, what the same block gives with NCCL all-reduces, and (within the tolerance of the one-GPU test) what the unsharded
block gives when the CPU oracle does the GEMMs.  Skipped on a box with one GPU."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def test_peer_all_reduce_equals_nccl(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29600 + os.getpid() % 300
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(HERE / "tp_two_rank_check.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("PEER_EQUALS_NCCL True") == 2, res.stdout[-2000:]
    assert res.stdout.count("FUSED_EQUALS_NCCL True") == 2, res.stdout[-2000:]
    assert res.stdout.count("AUTO_EQUALS_NCCL True") == 2, res.stdout[-2000:]
    assert res.stdout.count("MATCHES_UNSHARDED_ORACLE True") == 2, res.stdout[-2000:]
