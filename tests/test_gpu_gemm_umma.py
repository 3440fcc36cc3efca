"""tcgen05 route (M > 16): int32 bit-exact against the CPU oracle, fp16 epilogues within tolerance."""
import numpy as np
import pytest

from helpers import dev, planes_dev, rand_codes, run_gemm
from test_gpu_gemm_fp16 import check_close

pytestmark = pytest.mark.gpu

CASES = [
    # M, N, K, x_bits, w_bits, x_signed, w_signed
    (128, 256, 128, 8, 8, True, True),
    (128, 256, 512, 4, 4, False, False),
    (17, 64, 128, 8, 2, True, False),
    (100, 200, 384, 3, 5, True, True),
    (300, 520, 1152, 8, 4, True, False),
    (512, 1024, 4096, 2, 2, True, True),
    (256, 4096, 2048, 8, 8, False, False),
    (130, 72, 640, 6, 7, False, True),
    (128, 4096, 4096, 4, 4, False, False),   # the reference's CPU-checkable configuration (W4A4, unsigned)
    (128, 4096, 4096, 4, 4, True, True),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "M{}N{}K{}a{}w{}{}{}".format(*c[:5], "s" if c[5] else "u", "s" if c[6] else "u"))
def test_int32(abq, oracle, cuda, case):
    M, N, K, p, q, xs, ws = case
    rng = np.random.default_rng(sum(case[:5]))
    x, w = rand_codes(rng, M, K, p, xs), rand_codes(rng, N, K, q, ws)
    got, st = run_gemm(abq, planes_dev(oracle, x, p), planes_dev(oracle, w, q), M, N, K, x_bits=p, w_bits=q, x_signed=xs, w_signed=ws,
                       route=abq.ROUTE_I8_UMMA)
    want = oracle.gemm_values_blas(x, w)
    if M * N * K * p * q <= 1 << 27:
        assert np.array_equal(oracle.compute_ref(oracle.pack(w, q), oracle.pack(x, p), xs, ws), want)
    assert np.array_equal(got, want), f"{np.count_nonzero(got != want)} of {got.size} differ"


# one full-size prefill case (M = 512, LLaMA-7B shapes) for every width pair of the prefill sweep that has none above
WIDTH_CASES = [(512, 4096, 4096, 3, 3, True), (512, 4096, 4096, 5, 5, True), (512, 11008, 4096, 6, 6, False), (512, 4096, 11008, 7, 7, True),
               (512, 12288, 4096, 4, 2, False), (2048, 4096, 4096, 6, 2, True), (512, 4096, 4096, 2, 2, False), (512, 4096, 4096, 8, 8, True)]


@pytest.mark.parametrize("case", WIDTH_CASES, ids=lambda c: "M{}N{}K{}a{}w{}{}".format(*c[:5], "s" if c[5] else "u"))
def test_int32_full_size_per_width(abq, oracle, cuda, case):
    """WxAx for x = 2..8 plus W2A4 and W2A6 at prefill sizes: int32 bit for bit against the oracle's exact product, on the route the
    planner picks by itself, and the per-channel fp16 epilogue on the same operands."""
    M, N, K, p, q, signed = case
    rng = np.random.default_rng(sum(case[:5]))
    x, w = rand_codes(rng, M, K, p, signed), rand_codes(rng, N, K, q, signed)
    xp, wp = planes_dev(oracle, x, p), planes_dev(oracle, w, q)
    got, st = run_gemm(abq, xp, wp, M, N, K, x_bits=p, w_bits=q, x_signed=signed, w_signed=signed)
    assert st.route == abq.ROUTE_I8_UMMA
    want = oracle.gemm_values_blas(x, w)
    assert np.array_equal(got, want), f"{np.count_nonzero(got != want)} of {got.size} differ"
    # channel scales that keep every product inside the fp16 range whatever the widths (6-bit x 6-bit sums reach 1.6e7)
    scale = (rng.uniform(0.5, 1.0, size=N) * (30000.0 / max(1.0, float(np.abs(want).max())))).astype(np.float16)
    got16, _ = run_gemm(abq, xp, wp, M, N, K, x_bits=p, w_bits=q, x_signed=signed, w_signed=signed, out_fp16=True,
                        scale_mode=abq.SCALE_CHANNEL, w_scale=dev(scale))
    check_close(got16, want.astype(np.float64) * scale.astype(np.float64)[None, :])


def test_literal_reference_loop_on_sampled_rows(abq, oracle, cuda):
    """W4A4 128 x 4096 x 4096: the literal plane/bit loop on a sample of rows, the GPU result on all of them."""
    M, N, K, p, q = 128, 4096, 4096, 4, 4
    rng = np.random.default_rng(5)
    x, w = rand_codes(rng, M, K, p, False), rand_codes(rng, N, K, q, False)
    got, _ = run_gemm(abq, planes_dev(oracle, x, p), planes_dev(oracle, w, q), M, N, K, x_bits=p, w_bits=q, x_signed=False, w_signed=False)
    rows = [0, 63, 127]
    lit = oracle.compute_ref(oracle.pack(w, q), oracle.pack(x[rows], p), False, False)
    assert np.array_equal(got[rows], lit)
    assert np.array_equal(got, oracle.gemm_values_blas(x, w))


@pytest.mark.parametrize("M,N,K,q", [(64, 512, 1024, 4), (512, 4096, 4096, 2), (200, 1000, 2176, 8)])
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
                      x_scale=dev(xs), route=abq.ROUTE_I8_UMMA)
    ref = oracle.dequant_gemm(x, w, ws, None if wz is None else wz.astype(np.int32), xs, None)
    check_close(got, ref)


def test_tensor_compat_is_bit_exact(abq, oracle, cuda):
    M, N, K, p, q = 96, 384, 512, 8, 2
    rng = np.random.default_rng(3)
    x, w = rand_codes(rng, M, K, p, True), rand_codes(rng, N, K, q, True)
    scale = np.float16(0.0123)
    got, _ = run_gemm(abq, planes_dev(oracle, x, p), planes_dev(oracle, w, q), M, N, K, x_bits=p, w_bits=q, x_signed=True, w_signed=True,
                      out_fp16=True, scale_mode=abq.SCALE_TENSOR_COMPAT, C=dev(np.array([scale])), route=abq.ROUTE_I8_UMMA)
    want = oracle.dequant_tensor_compat(oracle.gemm_values_blas(x, w), scale)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("case", [(4096, 4096, 256, 4, 4, False, False), (1000, 12000, 384, 8, 3, True, False), (2100, 6000, 128, 2, 2, True, True)],
                         ids=lambda c: "M{}N{}K{}a{}w{}".format(*c[:5]))
def test_persistent_many_tiles_per_cta(abq, oracle, cuda, case):
    """More output tiles than three rounds of CTAs: every CTA reuses both TMEM accumulators and wraps its TMA ring
    across tile boundaries; ragged last tiles in both directions."""
    M, N, K, p, q, xs, ws = case
    rng = np.random.default_rng(M + N)
    x, w = rand_codes(rng, M, K, p, xs), rand_codes(rng, N, K, q, ws)
    got, st = run_gemm(abq, planes_dev(oracle, x, p), planes_dev(oracle, w, q), M, N, K, x_bits=p, w_bits=q, x_signed=xs, w_signed=ws,
                       route=abq.ROUTE_I8_UMMA)
    tiles = -(-M // 128) * -(-N // st.tile[0])
    assert tiles > 2 * st.grid[0], "meant to give every CTA several tiles"
    assert np.array_equal(got, oracle.gemm_values_blas(x, w))


def test_persistent_channel_parameters_follow_the_tile(abq, oracle, cuda):
    """Per-channel scale and zero point are staged per tile in two alternating shared-memory buffers: many tiles per CTA."""
    M, N, K, p, q = 2048, 6000, 256, 8, 4
    rng = np.random.default_rng(11)
    x, w = rand_codes(rng, M, K, p, True), rand_codes(rng, N, K, q, False)
    scale = rng.uniform(0.001, 0.02, size=N).astype(np.float16)
    zero = rng.integers(0, 1 << q, size=N, dtype=np.uint8)
    xs = rng.uniform(0.5, 2.0, size=M).astype(np.float32)
    got, _ = run_gemm(abq, planes_dev(oracle, x, p), planes_dev(oracle, w, q), M, N, K, x_bits=p, w_bits=q, x_signed=True, w_signed=False,
                      route=abq.ROUTE_I8_UMMA, out_fp16=True, scale_mode=abq.SCALE_CHANNEL, w_scale=dev(scale), w_zero=dev(zero), x_scale=dev(xs))
    acc = oracle.gemm_values_blas(x, w).astype(np.float64) - zero.astype(np.float64)[None, :] * x.sum(axis=1, dtype=np.int64)[:, None]
    check_close(got, acc * scale.astype(np.float64)[None, :] * xs.astype(np.float64)[:, None])


def test_full_size_prefill_rows_match_decode_route(abq, oracle, cuda):
    """W2A6 at a full prefill size (M=2048, N=11008, K=4096): blocks of 16 rows of the tcgen05 result equal, bit for bit,
    the mma.sync decode route on the same rows and the oracle's product of the code matrices."""
    M, N, K, p, q = 2048, 11008, 4096, 6, 2
    rng = np.random.default_rng(2048)
    x, w = rand_codes(rng, M, K, p, True), rand_codes(rng, N, K, q, False)
    wp = planes_dev(oracle, w, q)
    got, _ = run_gemm(abq, planes_dev(oracle, x, p), wp, M, N, K, x_bits=p, w_bits=q, x_signed=True, w_signed=False, route=abq.ROUTE_I8_UMMA)
    for r0 in (0, 1008, 2032):
        rows = slice(r0, r0 + 16)
        small, _ = run_gemm(abq, planes_dev(oracle, x[rows], p), wp, 16, N, K, x_bits=p, w_bits=q, x_signed=True, w_signed=False,
                            route=abq.ROUTE_I8_MMA)
        assert np.array_equal(got[rows], small)
        assert np.array_equal(small, oracle.gemm_values_blas(x[rows], w))
    # linearity over all rows: row sums of the result = (sum of the token codes) x W
    total = oracle.gemm_values_blas(x.sum(axis=0, dtype=np.int64)[None, :].astype(np.int64), w.astype(np.int64))
    assert np.array_equal(got.astype(np.int64).sum(axis=0)[None, :], total)


def test_prepared_weights_give_the_same_result(abq, oracle, cuda):
    """ABQ_FLAG_WEIGHTS_PREPARED: the weight codes are expanded once into the plan's workspace, later calls expand the
    activations only (new activations each call, same weights)."""
    import torch
    from abq_llm_b200 import binding as B
    M, N, K, p, q = 300, 1000, 1152, 8, 3
    rng = np.random.default_rng(9)
    w = rand_codes(rng, N, K, q, False)
    wp = planes_dev(oracle, w, q)
    ws = torch.empty(abq.gemm_workspace_bytes(M, N, K, p, q, abq.ROUTE_I8_UMMA), dtype=torch.uint8, device="cuda")
    out = torch.empty((M, N), dtype=torch.int32, device="cuda")
    xbuf = torch.empty((p, M, K // 32), dtype=torch.int32, device="cuda")
    prm = B.make_params(M, N, K, xbuf, wp, out, x_bits=p, w_bits=q, x_signed=True, w_signed=False, route=abq.ROUTE_I8_UMMA,
                        flags=abq.FLAG_WEIGHTS_PREPARED, workspace=ws)
    st = abq.gemm_init(prm)
    abq.gemm_prepare_weights(st)
    for i in range(3):
        x = rand_codes(rng, M, K, p, True)
        xbuf.copy_(planes_dev(oracle, x, p))
        abq.gemm_exec(st)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), oracle.gemm_values_blas(x, w)), f"call {i}"


GROUP_CASES = [
    # M, N, K, x_bits, x_signed, w_bits, w_signed, group, with_zero, expected route
    (40, 320, 1024, 8, True, 4, False, 128, True, "umma"),
    (300, 1000, 1152, 8, True, 2, False, 128, True, "umma"),
    (512, 4096, 4096, 8, True, 3, False, 128, True, "umma"),
    (130, 200, 2048, 8, True, 7, False, 256, True, "umma"),
    (200, 520, 1536, 4, False, 4, False, 128, False, "umma"),     # unsigned activations: conversion instruction path
    (64, 256, 1024, 8, True, 4, True, 128, False, "umma"),        # signed weights, no zero points
    (2048, 2048, 512, 8, True, 4, False, 128, True, "umma"),      # several tiles per CTA
    (100, 512, 4096, 8, True, 8, False, 128, True, "mma"),        # w - z does not fit int8: 16 rows per launch instead
    (33, 96, 1280, 8, True, 3, False, 640, True, "umma"),
    # scale groups of 64 features (two per K block): the W2A8 g64 configuration at LLaMA-2-13B widths, ragged tiles, 4-bit
    (40, 320, 1024, 8, True, 2, False, 64, True, "umma"),
    (300, 1000, 1152, 8, True, 4, False, 64, True, "umma"),
    (512, 5120, 5120, 8, True, 2, False, 64, True, "umma"),
    (256, 640, 13824, 8, True, 2, False, 64, True, "umma"),
    (200, 520, 1536, 4, False, 4, False, 64, False, "umma"),
]


@pytest.mark.parametrize("case", GROUP_CASES, ids=lambda c: "M{}N{}K{}a{}w{}g{}{}".format(c[0], c[1], c[2], c[3], c[5], c[7], "z" if c[8] else ""))
def test_per_group_scales_on_the_tensor_core_route(abq, oracle, cuda, case):
    """ABQ_SCALE_GROUP at prefill shapes: the accumulator is drained per scale group, zero points are folded into the
    int8 weight codes.  Against the oracle's float64 dequantised product."""
    M, N, K, p, xs, q, wsg, group, with_zero, want_route = case
    rng = np.random.default_rng(M + N + K + q)
    x = rand_codes(rng, M, K, p, xs)
    w = rand_codes(rng, N, K, q, wsg)
    G = K // group
    scale = rng.uniform(0.001, 0.02, size=(N, G)).astype(np.float16)
    zero = rng.integers(0, 1 << q, size=(N, G)).astype(np.uint8) if with_zero else None
    tok = rng.uniform(0.5, 2.0, size=M).astype(np.float32)
    got, st = run_gemm(abq, planes_dev(oracle, x, p), planes_dev(oracle, w, q), M, N, K, x_bits=p, w_bits=q, x_signed=xs, w_signed=wsg,
                       out_fp16=True, scale_mode=abq.SCALE_GROUP, group_size=group, w_scale=dev(scale), w_zero=None if zero is None else dev(zero),
                       x_scale=dev(tok))
    assert st.route == (abq.ROUTE_I8_UMMA if want_route == "umma" else abq.ROUTE_I8_MMA)
    ref = oracle.dequant_gemm(x, w, scale, None if zero is None else zero.astype(np.int32), tok, group)
    check_close(got, ref)


@pytest.mark.parametrize("case", [(130, 72, 640, 6, 7, False, True), (300, 520, 1152, 8, 4, True, False), (1000, 12000, 384, 8, 3, True, False),
                                  (4096, 4096, 256, 4, 4, False, False)], ids=lambda c: "M{}N{}K{}a{}w{}".format(*c[:5]))
def test_cta_pairs(abq, oracle, cuda, case, monkeypatch):
    """The cta_group::2 kernel (opt-in): a pair of CTAs per 256 x 256 tile, ragged tiles in both directions, a second
    CTA without rows, several tiles per pair.  int32 bit-exact, and the fp16 per-channel epilogue."""
    monkeypatch.setenv("ABQ_UMMA_PAIRS", "1")
    monkeypatch.setenv("ABQ_UMMA_BN", "256")   # small problems would otherwise get narrower, unpaired tiles
    M, N, K, p, q, xs, ws = case
    rng = np.random.default_rng(M * 3 + N)
    x, w = rand_codes(rng, M, K, p, xs), rand_codes(rng, N, K, q, ws)
    xp, wp = planes_dev(oracle, x, p), planes_dev(oracle, w, q)
    got, st = run_gemm(abq, xp, wp, M, N, K, x_bits=p, w_bits=q, x_signed=xs, w_signed=ws, route=abq.ROUTE_I8_UMMA)
    assert st.cluster == 2
    want = oracle.gemm_values_blas(x, w)
    assert np.array_equal(got, want)
    scale = rng.uniform(0.001, 0.02, size=N).astype(np.float16)
    got16, _ = run_gemm(abq, xp, wp, M, N, K, x_bits=p, w_bits=q, x_signed=xs, w_signed=ws, route=abq.ROUTE_I8_UMMA, out_fp16=True,
                        scale_mode=abq.SCALE_CHANNEL, w_scale=dev(scale))
    check_close(got16, want.astype(np.float64) * scale.astype(np.float64)[None, :])
