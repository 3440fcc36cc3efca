"""Bit-exact int32 parity of every GPU route against the CPU oracle (and the reference loop itself)."""
import numpy as np
import pytest

from helpers import planes_dev, rand_codes, run_gemm

pytestmark = pytest.mark.gpu

DECODE_CASES = [
    # M, N, K, x_bits, w_bits, x_signed, w_signed
    (1, 64, 128, 8, 2, True, False),
    (1, 256, 1024, 8, 2, True, True),
    (4, 192, 2048, 8, 3, True, False),
    (8, 320, 4096, 8, 4, True, True),
    (16, 128, 1152, 8, 4, True, False),
    (13, 100, 384, 4, 4, False, False),
    (5, 72, 1280, 3, 5, True, True),
    (16, 520, 2176, 8, 8, False, False),
    (2, 64, 640, 2, 2, True, True),
    (7, 48, 3200, 6, 7, False, True),
    (1, 4096, 4096, 8, 2, True, False),
    (16, 1024, 11008, 8, 4, True, True),
    (3, 200, 256, 1, 1, False, False),
    (37, 200, 640, 8, 3, True, False),      # taller than one launch of the mma.sync route: 16 rows per launch
    (48, 64, 11008, 8, 4, True, True),
]


@pytest.mark.parametrize("case", DECODE_CASES, ids=lambda c: "M{}N{}K{}a{}w{}{}{}".format(*c[:5], "s" if c[5] else "u", "s" if c[6] else "u"))
@pytest.mark.parametrize("route", ["i8_mma", "b1_mma"])
def test_int32_small_m(abq, oracle, cuda, case, route):
    M, N, K, p, q, xs, ws = case
    if route == "b1_mma" and N * K > 1 << 22:
        pytest.skip("the emulated 1-bit route is only cross-checked on small shapes")
    rng = np.random.default_rng(hash(case) & 0xffff)
    x = rand_codes(rng, M, K, p, xs)
    w = rand_codes(rng, N, K, q, ws)
    xp, wp = planes_dev(oracle, x, p), planes_dev(oracle, w, q)
    got, st = run_gemm(abq, xp, wp, M, N, K, x_bits=p, w_bits=q, x_signed=xs, w_signed=ws,
                       route=abq.ROUTE_I8_MMA if route == "i8_mma" else abq.ROUTE_B1_MMA)
    want = oracle.gemm_values_blas(x, w)
    if M * N * K * p * q <= 1 << 27:  # the literal plane/bit loop where it finishes in a blink
        lit = oracle.compute_ref(oracle.pack(w, q), oracle.pack(x, p), xs, ws)
        assert np.array_equal(lit, want)
    assert np.array_equal(got, want), f"{np.count_nonzero(got != want)} of {got.size} differ"


@pytest.mark.parametrize("one_shot", [False, True], ids=["plan_exec", "one_shot"])
def test_split_k_counters_on_dirty_workspace(abq, oracle, cuda, one_shot):
    """K split over CTAs (activation records of all of K do not fit one CTA): the arrival counters live in the
    caller's workspace, which here starts as garbage.  Planning (or the one-shot call) must clear them, and
    repeated launches of one plan must leave them ready for the next launch."""
    import torch
    from abq_llm_b200 import binding as B
    M, N, K, p, q = 16, 520, 11008, 8, 4
    rng = np.random.default_rng(77)
    x = rand_codes(rng, M, K, p, True)
    w = rand_codes(rng, N, K, q, False)
    xp, wp = planes_dev(oracle, x, p), planes_dev(oracle, w, q)
    want = oracle.gemm_values_blas(x, w)
    out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    ws = torch.full((max(256, abq.gemm_workspace_bytes(M, N, K, p, q, abq.ROUTE_I8_MMA)),), 0xA5, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    prm = B.make_params(M, N, K, xp, wp, out, x_bits=p, w_bits=q, x_signed=True, w_signed=False, route=abq.ROUTE_I8_MMA,
                        workspace=ws, status_word=status)
    torch.cuda.synchronize()
    if one_shot:
        for _ in range(3):
            out.fill_(-1)
            abq.gemm(prm)
            torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy(), want)
    else:
        st = abq.gemm_init(prm)
        assert st.cluster > 1, "this shape is meant to split K over CTAs"
        for _ in range(3):
            out.fill_(-1)
            abq.gemm_exec(st)
            torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy(), want)
    assert int(status.item()) == 0


def test_one_shot_plan_reuse(abq, oracle, cuda):
    """The one-shot entry keeps its plans per host thread.  The same parameter block again must give the same result, a block
    that differs only in its pointers must get its own plan, and more distinct blocks than the cache holds must still all be
    right (entries are replaced in turn)."""
    import torch
    from abq_llm_b200 import binding as B
    p, q, K, N = 8, 4, 1024, 72
    rng = np.random.default_rng(2024)
    cases = []
    for i in range(40):
        M = 1 + i % 5
        x = rand_codes(rng, M, K, p, True)
        w = rand_codes(rng, N, K, q, False)
        out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
        ws = torch.zeros(max(256, abq.gemm_workspace_bytes(M, N, K, p, q, abq.ROUTE_I8_MMA)), dtype=torch.uint8, device="cuda")
        xp, wp = planes_dev(oracle, x, p), planes_dev(oracle, w, q)
        prm = B.make_params(M, N, K, xp, wp, out, x_bits=p, w_bits=q, x_signed=True, w_signed=False, route=abq.ROUTE_I8_MMA, workspace=ws)
        cases.append((prm, out, oracle.gemm_values_blas(x, w), (xp, wp, ws)))
    for rounds in range(3):
        for prm, out, want, _ in cases:
            out.fill_(-1)
            abq.gemm(prm)
            abq.gemm(prm)
        torch.cuda.synchronize()
        for prm, out, want, _ in cases:
            assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("M,N,K,p,q,signed", [(1, 40, 128, 8, 2, True), (3, 96, 1152, 3, 5, False), (16, 72, 4096, 8, 2, True), (37, 64, 2176, 8, 8, True),
                                              (5, 200, 11008, 4, 4, False), (64, 48, 640, 2, 2, False), (9, 33, 1024, 7, 3, True), (130, 32, 256, 1, 1, False),
                                              (2, 4096, 4096, 8, 2, True), (20, 256, 1280, 6, 6, True)])
def test_plane_stacked_b1_route(abq, oracle, cuda, M, N, K, p, q, signed):
    """The 1-bit route with the planes stacked along the rows of both operands: widths that do not divide a tile of eight
    stacked rows (tokens straddling tiles), more tokens than one CTA takes, weight rows that do not fill the last CTA, a K
    that is not a whole number of 1024-feature stages."""
    rng = np.random.default_rng(M * 131 + N + K + p * 7 + q)
    x, w = rand_codes(rng, M, K, p, signed), rand_codes(rng, N, K, q, signed)
    got, _ = run_gemm(abq, planes_dev(oracle, x, p), planes_dev(oracle, w, q), M, N, K, x_bits=p, w_bits=q, x_signed=signed, w_signed=signed,
                      route=abq.ROUTE_B1_MMA)
    assert np.array_equal(got, oracle.gemm_values_blas(x, w))
