"""Fused dequantisation epilogues (fp16 output).

Tolerance: the kernels accumulate in int32 inside a scale group and in fp32 across groups, then round
once to fp16.  Against the double-precision oracle that is at most half an fp16 ulp of the result plus
fp32 summation error, bounded here as |got - ref| <= 2^-10 * |ref| + 2^-11 * max|ref| (fp16 has an
11-bit significand).  The reference-compatible per-tensor mode is integer-exact up to its two fp16
roundings and is compared bit for bit.
"""
import numpy as np
import pytest

from helpers import dev, planes_dev, rand_codes, run_gemm

pytestmark = pytest.mark.gpu


def check_close(got, ref):
    got = got.astype(np.float64)
    bound = 2.0 ** -10 * np.abs(ref) + 2.0 ** -11 * np.abs(ref).max()
    err = np.abs(got - ref)
    assert np.all(err <= bound), f"max abs err {err.max():.4g}, max rel {np.max(err / (np.abs(ref) + 1e-9)):.4g}"


@pytest.mark.parametrize("route", ["i8_mma", "b1_mma"])
@pytest.mark.parametrize("M,N,K,p,q,signed", [(1, 256, 512, 8, 2, True), (8, 96, 4096, 8, 2, False), (16, 4096, 1024, 8, 2, True)])
def test_tensor_compat_is_bit_exact(abq, oracle, cuda, route, M, N, K, p, q, signed):
    rng = np.random.default_rng(M + N + K)
    x, w = rand_codes(rng, M, K, p, signed), rand_codes(rng, N, K, q, signed)
    scale = np.float16(0.0123)
    got, _ = run_gemm(abq, planes_dev(oracle, x, p), planes_dev(oracle, w, q), M, N, K, x_bits=p, w_bits=q, x_signed=signed,
                      w_signed=signed, out_fp16=True, scale_mode=abq.SCALE_TENSOR_COMPAT, C=dev(np.array([scale])),
                      route=abq.ROUTE_I8_MMA if route == "i8_mma" else abq.ROUTE_B1_MMA)
    want = oracle.dequant_tensor_compat(oracle.gemm_values_blas(x, w), scale)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("M,N,K,q", [(1, 4096, 4096, 2), (4, 1024, 4096, 3), (16, 512, 11008, 4), (7, 200, 1152, 4), (1, 64, 128, 8)])
@pytest.mark.parametrize("with_zero", [False, True])
def test_per_channel(abq, oracle, cuda, M, N, K, q, with_zero):
    rng = np.random.default_rng(N + K + q)
    x = np.clip(np.rint(rng.normal(0, 30, size=(M, K))), -128, 127).astype(np.int32)
    w = rand_codes(rng, N, K, q, False)
    ws = rng.uniform(0.001, 0.02, size=N).astype(np.float16)
    wz = rng.integers(0, 1 << q, size=N).astype(np.uint8) if with_zero else None
    xs = rng.uniform(0.01, 0.05, size=M).astype(np.float32)
    got, _ = run_gemm(abq, planes_dev(oracle, x, 8), planes_dev(oracle, w, q), M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False,
                      out_fp16=True, scale_mode=abq.SCALE_CHANNEL, w_scale=dev(ws), w_zero=None if wz is None else dev(wz),
                      x_scale=dev(xs), route=abq.ROUTE_I8_MMA)
    ref = oracle.dequant_gemm(x, w, ws, None if wz is None else wz.astype(np.int32), xs, None)
    check_close(got, ref)


@pytest.mark.parametrize("M,N,K,q,group", [(1, 4096, 4096, 2, 128), (4, 512, 4096, 3, 128), (16, 320, 11008, 4, 128), (8, 128, 2048, 4, 256),
                                           (3, 64, 1536, 2, 384), (16, 4096, 4096, 4, 128),
                                           (40, 320, 1024, 4, 128), (100, 512, 4096, 2, 128), (33, 96, 11008, 3, 256)])
@pytest.mark.parametrize("w_signed", [False, True])
def test_per_group(abq, oracle, cuda, M, N, K, q, group, w_signed):
    rng = np.random.default_rng(N + K + q + group)
    x = np.clip(np.rint(rng.normal(0, 30, size=(M, K))), -128, 127).astype(np.int32)
    w = rand_codes(rng, N, K, q, w_signed)
    G = K // group
    ws = rng.uniform(0.001, 0.02, size=(N, G)).astype(np.float16)
    wz = rng.integers(0, 1 << q, size=(N, G)).astype(np.uint8)
    got, st = run_gemm(abq, planes_dev(oracle, x, 8), planes_dev(oracle, w, q), M, N, K, x_bits=8, w_bits=q, x_signed=True,
                       w_signed=w_signed, out_fp16=True, scale_mode=abq.SCALE_GROUP, group_size=group, w_scale=dev(ws), w_zero=dev(wz),
                       route=abq.ROUTE_I8_MMA)  # taller than 16 rows: one launch per 16 rows
    assert st.route == abq.ROUTE_I8_MMA
    ref = oracle.dequant_gemm(x, w, ws, wz.astype(np.int32), None, group)
    check_close(got, ref)


@pytest.mark.parametrize("N,K", [(4096, 4096), (12288, 4096), (11008, 4096), (4096, 11008)])
@pytest.mark.parametrize("q", [2, 3, 4])
def test_full_size_sweep_shapes(abq, oracle, cuda, N, K, q):
    """All 36 GEMMs the benchmark times, at full size (LLaMA-7B shapes, W{2,3,4}A8, M in {1, 4, 16}, g128 scale + zero point, int8
    activations ~N(0, 30)): fp16 result against the oracle's float64 dequantised product, and the int32 accumulation bit for
    bit.  One weight matrix per (shape, width), the three token counts on it."""
    rng = np.random.default_rng(N + K + q)
    w = rand_codes(rng, N, K, q, False)
    ws = rng.uniform(0.001, 0.02, size=(N, K // 128)).astype(np.float16)
    wz = rng.integers(0, 1 << q, size=(N, K // 128)).astype(np.uint8)
    wp, dws, dwz = planes_dev(oracle, w, q), dev(ws), dev(wz)
    for M in (1, 4, 16):
        x = np.clip(np.rint(rng.normal(0, 30, size=(M, K))), -128, 127).astype(np.int32)
        xp = planes_dev(oracle, x, 8)
        got, _ = run_gemm(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False, out_fp16=True, scale_mode=abq.SCALE_GROUP,
                          group_size=128, w_scale=dws, w_zero=dwz, flags=abq.FLAG_PDL)
        check_close(got, oracle.dequant_gemm(x, w, ws, wz.astype(np.int32), None, 128))
        acc, _ = run_gemm(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False)
        assert np.array_equal(acc, oracle.gemm_values_blas(x, w)), f"M={M}"
