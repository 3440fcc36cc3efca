"""Tensor-parallel block linears on CPU: two gloo ranks with a numpy stand-in for the GEMMs (the oracle), checking the
shard ranges, that column/row slices of planes, scales and zero points line up, and that the all-reduced result equals
the same computation done rank by rank in one process."""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _tp():
    spec = importlib.util.spec_from_file_location("tp_linear_under_test", ROOT / "abq-llm_b200" / "tp_linear.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


class NumpyBackend:
    """GEMMs through the CPU oracle; the all-reduce through torch.distributed when given."""

    def __init__(self, group, dist_mod=None, x_scale=16.0):
        from oracle import oracle as O
        self.O, self.group, self.dist, self.x_scale = O, group, dist_mod, x_scale

    def make_linear(self, codes, scale, zero, w_bits, group, reduce_output=False):
        be = self

        class L:
            out_features, in_features = codes.shape

            def __call__(self, x):
                _, q = be.O.quantize_half_compat(np.ascontiguousarray(x, dtype=np.float16), be.x_scale, 8)
                q = ((q + 128) % 256) - 128  # the low 8 bits, as the planes hold them
                z = None if zero is None else zero.astype(np.int32)
                ref = be.O.dequant_gemm(q, codes, scale if group else scale[:, None], z if (z is None or group) else z[:, None],
                                        None, group if group else self.in_features)
                return (ref / be.x_scale).astype(np.float16)
        return L()

    def all_reduce(self, t):
        if self.dist is not None:
            tt = torch.from_numpy(t)
            self.dist.all_reduce(tt)
        return t

    def glue_attention(self, qkv, hl, out=None):
        return np.ascontiguousarray(qkv[:, :hl])

    def glue_residual(self, a, b, out=None):
        return (a + b).astype(np.float16)

    def glue_swiglu(self, gu, fl, out=None):
        g = gu[:, :fl].astype(np.float32)
        return (g / (1 + np.exp(-g)) * gu[:, fl:].astype(np.float32)).astype(np.float16)


def _weights(tp, hidden, ffn, q, group, seed=3):
    rng = np.random.default_rng(seed)
    out = []
    for spec in tp.llama_block_specs(hidden, ffn):
        codes = rng.integers(0, 1 << q, size=(spec.out_features, spec.in_features), dtype=np.int32)
        G = spec.in_features // group if group else 1
        scale = rng.uniform(0.001, 0.01, size=(spec.out_features, G) if group else (spec.out_features,)).astype(np.float16)
        zero = rng.integers(0, 1 << q, size=scale.shape, dtype=np.uint8)
        out.append((codes, scale, zero))
    return out


HIDDEN, FFN, Q, GROUP, M = 256, 640, 4, 128, 3


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tp = _tp()
    block = tp.TensorParallelBlockLinears(NumpyBackend(GROUP, dist), HIDDEN, FFN, rank, world, _weights(tp, HIDDEN, FFN, Q, GROUP), Q, GROUP)
    x = np.random.default_rng(1).normal(0, 1.0, size=(M, HIDDEN)).astype(np.float16)
    y = block.forward(x)
    dist.barrier()
    out.put((rank, y))
    dist.destroy_process_group()


def test_two_ranks_match_the_rank_by_rank_computation():
    tp = _tp()
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(out.get() for _ in range(2))
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert np.array_equal(got[0], got[1]), "the result is replicated"

    # the same thing without processes: partial results of both ranks, summed in fp16 in rank order
    weights = _weights(tp, HIDDEN, FFN, Q, GROUP)

    class Collect(NumpyBackend):
        pass
    blocks = [tp.TensorParallelBlockLinears(Collect(GROUP), HIDDEN, FFN, r, 2, weights, Q, GROUP) for r in range(2)]
    x = np.random.default_rng(1).normal(0, 1.0, size=(M, HIDDEN)).astype(np.float16)
    be = blocks[0].backend
    o = sum_fp16([b.layers["o"](be.glue_attention(b.layers["qkv"](x), b.layers["qkv"].out_features // 3)) for b in blocks])
    h = be.glue_residual(x, o)
    d = sum_fp16([b.layers["down"](be.glue_swiglu(b.layers["gate_up"](h), b.layers["gate_up"].out_features // 2)) for b in blocks])
    want = be.glue_residual(h, d)
    assert np.array_equal(got[0], want)


def sum_fp16(parts):
    acc = parts[0].copy()
    for p in parts[1:]:
        acc = (torch.from_numpy(acc) + torch.from_numpy(p)).numpy()
    return acc


def test_shard_ranges():
    tp = _tp()
    assert tp.unit_ranges(11008, 4) == [(0, 2816), (2816, 5632), (5632, 8320), (8320, 11008)]   # 22/22/21/21 units of 128
    assert tp.unit_ranges(13824, 8)[-1] == (13824 - 13 * 128, 13824)                             # 14/14/14/14/13/13/13/13
    assert [e - b for b, e in tp.unit_ranges(4096, 8)] == [512] * 8
    with pytest.raises(ValueError):
        tp.unit_ranges(4100, 2)
    specs = {s.name: s for s in tp.llama_block_specs(4096, 11008)}
    rows, cols = tp.shard_of(specs["gate_up"], 3, 4)
    assert len(rows) == 2 * (11008 - 8320) and rows[0] == 8320 and rows[len(rows) // 2] == 11008 + 8320
    rows, cols = tp.shard_of(specs["down"], 3, 4)
    assert (cols.start, cols.stop) == (8320, 11008)   # the K slice of `down` is the feature slice `gate_up` produced
