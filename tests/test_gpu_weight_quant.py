"""Quantise-on-load (abq_quantize_weights_half) against the oracle's float32 restatement of the reference's weight
quantiser, bit for bit: codes (read back out of the planes), fp16 scales, zero points.  Then the packer: shards written in
the reference loader's file layout, read back, multiplied on the GPU, equal to the unsharded product."""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import dev, planes_dev, run_gemm
from test_gpu_gemm_fp16 import check_close

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("N,K,bits,group,symmetric", [(64, 512, 4, 0, False), (200, 1024, 2, 64, False), (96, 4096, 3, 128, False),
                                                      (33, 11008, 4, 128, False), (128, 2048, 8, 256, False), (40, 640, 4, 128, True),
                                                      (16, 128, 1, 32, False), (4096, 4096, 4, 0, False), (256, 5120, 2, 64, False)])
def test_matches_the_oracle_quantiser(abq, oracle, cuda, N, K, bits, group, symmetric):
    rng = np.random.default_rng(N + K + bits)
    w = (rng.normal(0, 0.02, size=(N, K)) + rng.normal(0, 0.005, size=(N, 1))).astype(np.float16)
    G = K // group if group else 1
    planes = torch.zeros((bits, N, K // 32), dtype=torch.int32, device="cuda")
    scale = torch.zeros((N, G), dtype=torch.float16, device="cuda")
    zero = torch.zeros((N, G), dtype=torch.uint8, device="cuda")
    abq.quantize_weights_half(dev(w), planes, scale, zero, N, K, bits, group, symmetric)
    torch.cuda.synchronize()
    want_codes, want_scale, want_zero = oracle.quantize_weights_minmax(w, bits, group or None, symmetric)
    got_codes = oracle.unpack(planes.cpu().numpy().view(np.uint32), False)
    assert np.array_equal(scale.cpu().numpy().view(np.uint16), want_scale.reshape(N, G).view(np.uint16))
    assert np.array_equal(zero.cpu().numpy(), want_zero.reshape(N, G))
    assert np.array_equal(got_codes, want_codes), f"{np.count_nonzero(got_codes != want_codes)} of {got_codes.size} codes differ"


def test_rejected_arguments(abq, cuda):
    w = torch.zeros((16, 128), dtype=torch.float16, device="cuda")
    planes = torch.zeros((4, 16, 4), dtype=torch.int32, device="cuda")
    s = torch.zeros(16, dtype=torch.float16, device="cuda")
    z = torch.zeros(16, dtype=torch.uint8, device="cuda")
    for kw in (dict(group_size=48), dict(group_size=96), dict(bits=9), dict(bits=1, symmetric=True)):
        args = dict(bits=4, group_size=0, symmetric=False)
        args.update(kw)
        with pytest.raises(abq.AbqError):
            abq.quantize_weights_half(w, planes, s, z, 16, 128, args["bits"], args["group_size"], args["symmetric"])


def test_shards_written_read_and_multiplied(abq, oracle, cuda, tmp_path):
    """fp16 weight -> quantise on the GPU -> per-rank files in the reference's layout -> read back -> the ranks' GEMMs
    (row-parallel: partial sums added) equal the GEMM on the unsharded quantised weight."""
    spec = importlib.util.spec_from_file_location("weight_files_gpu", ROOT / "abq-llm_b200" / "weight_files.py")
    wf = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = wf
    spec.loader.exec_module(wf)
    rng = np.random.default_rng(4)
    hidden, ffn, tp, q, group, M = 512, 1408, 4, 4, 128, 5   # 1408 = 11 units of 128: uneven 3/3/3/2 split
    x = np.clip(np.rint(rng.normal(0, 30, size=(M, ffn))), -128, 127).astype(np.int32)
    w = rng.normal(0, 0.02, size=(hidden, ffn)).astype(np.float16)
    shards = wf.quantize_and_shard(abq, torch, dev(w), "mlp.down_proj", tp, q, group)
    for r, (p, s, z) in enumerate(shards):
        wf.write_shard(tmp_path, 0, "mlp.down_proj", r, p, s, z)
    codes, scale, zero = oracle.quantize_weights_minmax(w, q, group)
    want = oracle.dequant_gemm(x, codes, scale, zero.astype(np.int32), None, group)
    total = np.zeros((M, hidden), dtype=np.float64)
    for r, (b, e) in enumerate(wf.split_ranges(ffn, tp, 128)):
        p, s, z = wf.read_shard(tmp_path, 0, "mlp.down_proj", r, q, hidden, e - b, groups=(e - b) // group)
        assert np.array_equal(oracle.unpack(p, False), codes[:, b:e])
        got, _ = run_gemm(abq, planes_dev(oracle, x[:, b:e], 8), dev(p.view(np.int32)), M, hidden, e - b, x_bits=8, w_bits=q, x_signed=True,
                          w_signed=False, out_fp16=True, scale_mode=abq.SCALE_GROUP, group_size=group, w_scale=dev(s), w_zero=dev(z))
        total += got.astype(np.float64)
    err = np.abs(total - want)
    assert np.all(err <= tp * (2.0 ** -10 * np.abs(want) + 2.0 ** -11 * np.abs(want).max()))
    # column-parallel: the ranks' output rows are the fused parts' slices
    wq = rng.normal(0, 0.02, size=(3 * hidden, hidden)).astype(np.float16)
    col = wf.quantize_and_shard(abq, torch, dev(wq), "attention.query_key_value", 2, 2, 0)
    cq, _, _ = oracle.quantize_weights_minmax(wq, 2, None)
    rows1 = np.concatenate([np.arange(pp * hidden + hidden // 2, (pp + 1) * hidden) for pp in range(3)])
    assert np.array_equal(oracle.unpack(col[1][0], False), cq[rows1])
