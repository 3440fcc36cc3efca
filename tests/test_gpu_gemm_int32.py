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
