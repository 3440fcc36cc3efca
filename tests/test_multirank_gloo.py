"""The N > 1 path of the benchmark on CPU: two gloo ranks.  The GEMM sweep does not shard (replicas only), so what
several ranks share is the rendezvous, the max-over-ranks timing rule and the whole-job aggregation."""
import importlib.util
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    bench = _bench()
    ms_local = 10.0 + 5.0 * rank                      # rank 1 is the slow one
    ms = bench.max_over_ranks(torch, dist, ms_local, "cpu")
    rate = bench.whole_job_rate(world, 1e9, 4, ms)    # 1 GB per rank and step, 4 steps
    dist.barrier()
    if rank == 0:
        out.put((ms, rate))
    dist.destroy_process_group()


def test_two_ranks_report_the_slowest_rank_and_the_whole_job():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    ms, rate = out.get()
    assert ms == 15.0
    assert rate == pytest.approx(2 * 1e9 * 4 / 15e-3)


def test_single_rank_is_the_identity():
    bench = _bench()
    assert bench.max_over_ranks(torch, None, 7.5, "cpu") == 7.5
    assert bench.algorithmic_bytes(1, 4096, 4096, 8, 2) == 4599808      # the worked example of the scope table
    assert bench.algorithmic_bytes(1, 11008, 4096, 8, 4) == 23627264
