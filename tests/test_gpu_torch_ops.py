"""The torch operators (abq_b200::gemm_planes, abq_b200::linear_half) and the reference extension's mul_w2a8 entry point
(algorithm/ABQ/csrc/ABQ_cuda.cu:24-53) against the oracle."""
import numpy as np
import pytest
import torch

from helpers import planes_dev, rand_codes

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(abq):
    import importlib
    return importlib.import_module("abq_llm_b200.torch_ops")


@pytest.mark.parametrize("M,N,K,p,q,signed", [(1, 512, 1024, 8, 2, True), (16, 200, 1152, 4, 4, False), (192, 256, 512, 8, 3, True)])
def test_gemm_planes_op(abq, oracle, cuda, ops, M, N, K, p, q, signed):
    rng = np.random.default_rng(M * 7 + q)
    x, w = rand_codes(rng, M, K, p, signed), rand_codes(rng, N, K, q, signed)
    got = torch.ops.abq_b200.gemm_planes(planes_dev(oracle, x, p), planes_dev(oracle, w, q), p, q, signed)
    torch.cuda.synchronize()
    assert got.dtype == torch.int32 and tuple(got.shape) == (M, N)
    assert np.array_equal(got.cpu().numpy(), oracle.gemm_values_blas(x, w))


@pytest.mark.parametrize("M,N,K,q,group", [(1, 512, 1024, 4, 0), (5, 264, 1152, 2, 128), (40, 128, 512, 4, 0)])
def test_linear_half_op(abq, oracle, cuda, ops, M, N, K, q, group):
    rng = np.random.default_rng(N + q)
    x = rng.normal(0, 1.5, size=(M, K)).astype(np.float16)
    w = rand_codes(rng, N, K, q, False)
    shape = (N, K // group) if group else (N,)
    scale = rng.uniform(0.001, 0.02, size=shape).astype(np.float16)
    zero = rng.integers(0, 1 << q, size=shape).astype(np.uint8)
    qs = 11.0
    got = torch.ops.abq_b200.linear_half(torch.from_numpy(x).cuda(), planes_dev(oracle, w, q), torch.from_numpy(scale).cuda(), torch.from_numpy(zero).cuda(),
                                         torch.full((1,), qs, dtype=torch.float32, device="cuda"), 8, q, group)
    torch.cuda.synchronize()
    _, codes = oracle.quantize_half_compat(x, qs, 8)
    codes = ((codes + 128) % 256) - 128
    want = oracle.dequant_gemm(codes, w, scale, zero, np.full(M, np.float32(1.0) / np.float32(qs), dtype=np.float32), group=group or None)
    got = got.cpu().numpy().astype(np.float64)
    # the tolerance of the fused epilogues (test_gpu_gemm_fp16.py): half an fp16 ulp of the result plus fp32 summation error
    bound = 2.0 ** -10 * np.abs(want) + 2.0 ** -11 * np.abs(want).max()
    assert np.all(np.abs(got - want) <= bound), float(np.max(np.abs(got - want) / bound))


def test_mul_w2a8_entry_point(abq, oracle, cuda, ops):
    M, N, K = 4, 384, 1024
    rng = np.random.default_rng(5)
    x, w = rand_codes(rng, M, K, 8, True), rand_codes(rng, N, K, 2, True)
    out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    ops.mul_w2a8(planes_dev(oracle, x, 8), planes_dev(oracle, w, 2), out, M, N, K)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.gemm_values_blas(x, w))
    with pytest.raises(RuntimeError, match="prob_k < 128"):
        ops.mul_w2a8(out, out, out, 1, 1, 64)
