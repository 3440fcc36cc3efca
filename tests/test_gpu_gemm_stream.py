"""Decode route over prepared weights (ABQ_FLAG_WEIGHTS_PREPARED + w_prepared: the planes re-ordered once at load time).

Same bar as the plane path: int32 bit for bit against the oracle's exact product, the reference-compatible fp16 mode bit
for bit, per-channel / per-group fp16 within the tolerance stated in test_gpu_gemm_fp16.py of the oracle's float64
dequantised product.  The prepared copy is made by the library from the reference's plane format, which stays the input."""
import numpy as np
import pytest
import torch

from helpers import dev, planes_dev, rand_codes
from test_gpu_gemm_fp16 import check_close

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def heuristic_plans(monkeypatch):
    """The tuning table sends some shapes to the kernel that reads the planes; these tests are about the prepared-weights
    kernel, so they plan with the heuristic alone (one test below checks that a table entry is honoured)."""
    monkeypatch.setenv("ABQ_TUNE_IGNORE", "1")


def run_prepared(abq, xp, wp, M, N, K, *, x_bits, w_bits, x_signed, w_signed, out_fp16=False, scale_mode=0, group_size=0, C=None,
                 w_scale=None, w_zero=None, x_scale=None, flags=0, x_quant_scale=None, calls=1):
    from abq_llm_b200 import binding as B
    out = torch.full((M, N), -7, dtype=torch.float16 if out_fp16 else torch.int32, device="cuda")
    ws = torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, x_bits, w_bits, abq.ROUTE_I8_MMA)), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = B.make_params(M, N, K, xp, wp, out, x_bits=x_bits, w_bits=w_bits, x_signed=x_signed, w_signed=w_signed,
                      out_dtype=abq.OUT_FP16 if out_fp16 else abq.OUT_INT32, scale_mode=scale_mode, group_size=group_size, C=C,
                      w_scale=w_scale, w_zero=w_zero, x_scale=x_scale, route=abq.ROUTE_I8_MMA, flags=flags | abq.FLAG_WEIGHTS_PREPARED,
                      workspace=ws, status_word=status, x_quant_scale=x_quant_scale)
    nbytes = abq.gemm_prepared_weight_bytes(p)
    assert nbytes >= w_bits * N * K // 8
    prepared = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    p.w_prepared = prepared.data_ptr()
    st = abq.gemm_init(p)
    abq.gemm_prepare_weights(st)
    torch.cuda.synchronize()
    for _ in range(calls):
        abq.gemm_exec(st)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device status word {int(status.item())}"
    return out.cpu().numpy(), st


INT_CASES = [
    # M, N, K, x_bits, w_bits, x_signed, w_signed
    (1, 4096, 4096, 8, 2, True, False), (1, 48, 128, 8, 2, True, True), (2, 200, 1152, 8, 3, True, False), (3, 520, 640, 4, 4, False, False),
    (4, 1000, 2048, 8, 4, True, True), (5, 72, 384, 6, 3, True, True), (8, 4096, 1024, 8, 8, True, True), (9, 136, 1152, 7, 2, False, False),
    (16, 512, 4096, 8, 4, True, False), (16, 1024, 11008, 8, 3, True, False), (20, 96, 2176, 8, 2, True, True), (33, 320, 1280, 8, 8, True, False),
    (1, 11008, 4096, 8, 3, True, False), (7, 4096, 11008, 8, 4, True, False), (1, 16, 128, 1, 2, False, False), (12, 4096, 4096, 3, 3, True, True),
]


@pytest.mark.parametrize("case", INT_CASES, ids=lambda c: "M{}N{}K{}a{}w{}{}{}".format(*c[:5], "s" if c[5] else "u", "s" if c[6] else "u"))
def test_int32_bit_exact(abq, oracle, cuda, case):
    M, N, K, p, q, xs, ws = case
    rng = np.random.default_rng(sum(case[:5]))
    x, w = rand_codes(rng, M, K, p, xs), rand_codes(rng, N, K, q, ws)
    got, st = run_prepared(abq, planes_dev(oracle, x, p), planes_dev(oracle, w, q), M, N, K, x_bits=p, w_bits=q, x_signed=xs, w_signed=ws, calls=2)
    want = oracle.gemm_values_blas(x, w)
    if M * N * K * p * q <= 1 << 26:
        assert np.array_equal(oracle.compute_ref(oracle.pack(w, q), oracle.pack(x, p), xs, ws), want)
    assert np.array_equal(got, want), f"{np.count_nonzero(got != want)} of {got.size} differ"


@pytest.mark.parametrize("env", [{"ABQ_STREAM_FULL": "1"}, {"ABQ_STREAM_MP": "8", "ABQ_STREAM_RING": "2"}, {"ABQ_STREAM_SLICES": "3"},
                                 {"ABQ_STREAM_WARPS": "4", "ABQ_STREAM_CTAS": "37"}, {"ABQ_STREAM_WARPS": "16", "ABQ_STREAM_FULL": "1", "ABQ_STREAM_CTAS": "296"}],
                         ids=lambda e: ",".join(f"{k[11:]}={v}" for k, v in e.items()))
@pytest.mark.parametrize("M,q", [(1, 2), (4, 3), (8, 4), (16, 2)])
def test_plan_variants(abq, oracle, cuda, monkeypatch, env, M, q):
    """Other launch shapes than the planner's default (one CTA per SM, deeper / shallower rings, K split over CTAs, fewer
    or more CTAs and warps): the same bits."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    N, K = 1512, 2688
    rng = np.random.default_rng(M + q)
    x, w = rand_codes(rng, M, K, 8, True), rand_codes(rng, N, K, q, False)
    xp, wp = planes_dev(oracle, x, 8), planes_dev(oracle, w, q)
    got, st = run_prepared(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False, calls=2)
    assert np.array_equal(got, oracle.gemm_values_blas(x, w))
    scale = rng.uniform(0.001, 0.02, size=(N, K // 128)).astype(np.float16)
    zero = rng.integers(0, 1 << q, size=(N, K // 128)).astype(np.uint8)
    got16, _ = run_prepared(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False, out_fp16=True, scale_mode=abq.SCALE_GROUP,
                            group_size=128, w_scale=dev(scale), w_zero=dev(zero), calls=2)
    check_close(got16, oracle.dequant_gemm(x, w, scale, zero.astype(np.int32), None, 128))


@pytest.mark.parametrize("M,N,K,q,group", [(1, 4096, 4096, 2, 128), (2, 512, 4096, 3, 128), (4, 320, 11008, 4, 128), (8, 128, 2048, 4, 256),
                                           (3, 64, 1536, 2, 384), (16, 4096, 4096, 4, 128), (1, 72, 1152, 8, 128), (5, 200, 640, 3, 128),
                                           (40, 320, 1024, 4, 128), (33, 96, 11008, 3, 256), (16, 512, 11008, 2, 128), (1, 4096, 11008, 3, 128)])
@pytest.mark.parametrize("w_signed", [False, True])
def test_per_group(abq, oracle, cuda, M, N, K, q, group, w_signed):
    rng = np.random.default_rng(N + K + q + group)
    x = np.clip(np.rint(rng.normal(0, 30, size=(M, K))), -128, 127).astype(np.int32)
    w = rand_codes(rng, N, K, q, w_signed)
    G = K // group
    ws = rng.uniform(0.001, 0.02, size=(N, G)).astype(np.float16)
    wz = rng.integers(0, 1 << q, size=(N, G)).astype(np.uint8)
    xs = rng.uniform(0.5, 2.0, size=M).astype(np.float32)
    got, st = run_prepared(abq, planes_dev(oracle, x, 8), planes_dev(oracle, w, q), M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=w_signed,
                           out_fp16=True, scale_mode=abq.SCALE_GROUP, group_size=group, w_scale=dev(ws), w_zero=dev(wz), x_scale=dev(xs), calls=2)
    check_close(got, oracle.dequant_gemm(x, w, ws, wz.astype(np.int32), xs, group))


@pytest.mark.parametrize("M,N,K,q,group", [(1, 4096, 4096, 2, 64), (2, 512, 1024, 3, 64), (4, 320, 2176, 4, 64), (8, 136, 640, 8, 64), (16, 1024, 4096, 2, 64),
                                           (33, 96, 1280, 3, 64), (5, 200, 1152, 4, 192), (16, 5120, 5120, 2, 64), (16, 5120, 13824, 2, 64),
                                           (1, 13824, 5120, 2, 64), (3, 15360, 5120, 2, 64)])
@pytest.mark.parametrize("w_signed", [False, True])
def test_scale_groups_of_64(abq, oracle, cuda, M, N, K, q, group, w_signed):
    """Scale groups that are an odd multiple of 64 features wide (the LLaMA-2-13B W2A8 g64 configuration: hidden 5120, FFN 13824):
    the prepared layout then uses 64-feature units."""
    rng = np.random.default_rng(N + K + q + group + M)
    x = np.clip(np.rint(rng.normal(0, 30, size=(M, K))), -128, 127).astype(np.int32)
    w = rand_codes(rng, N, K, q, w_signed)
    G = K // group
    ws = rng.uniform(0.001, 0.02, size=(N, G)).astype(np.float16)
    wz = rng.integers(0, 1 << q, size=(N, G)).astype(np.uint8)
    got, st = run_prepared(abq, planes_dev(oracle, x, 8), planes_dev(oracle, w, q), M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=w_signed,
                           out_fp16=True, scale_mode=abq.SCALE_GROUP, group_size=group, w_scale=dev(ws), w_zero=dev(wz), calls=2)
    check_close(got, oracle.dequant_gemm(x, w, ws, wz.astype(np.int32), None, group))


@pytest.mark.parametrize("M,N,K,q", [(1, 4096, 4096, 2), (4, 1024, 4096, 3), (16, 512, 11008, 4), (7, 200, 1152, 4), (1, 64, 128, 8)])
@pytest.mark.parametrize("with_zero", [False, True])
def test_per_channel_and_tensor_compat(abq, oracle, cuda, M, N, K, q, with_zero):
    rng = np.random.default_rng(N + K + q)
    x = np.clip(np.rint(rng.normal(0, 30, size=(M, K))), -128, 127).astype(np.int32)
    w = rand_codes(rng, N, K, q, False)
    ws = rng.uniform(0.001, 0.02, size=N).astype(np.float16)
    wz = rng.integers(0, 1 << q, size=N).astype(np.uint8) if with_zero else None
    xs = rng.uniform(0.01, 0.05, size=M).astype(np.float32)
    xp, wp = planes_dev(oracle, x, 8), planes_dev(oracle, w, q)
    got, _ = run_prepared(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False, out_fp16=True, scale_mode=abq.SCALE_CHANNEL,
                          w_scale=dev(ws), w_zero=None if wz is None else dev(wz), x_scale=dev(xs))
    check_close(got, oracle.dequant_gemm(x, w, ws, None if wz is None else wz.astype(np.int32), xs, None))
    if not with_zero:
        scale = np.float16(0.0123)
        got, _ = run_prepared(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False, out_fp16=True,
                              scale_mode=abq.SCALE_TENSOR_COMPAT, C=dev(np.array([scale])))
        want = oracle.dequant_tensor_compat(oracle.gemm_values_blas(x, w), scale)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("M,N,K,q", [(1, 1024, 4096, 2), (6, 320, 1152, 4), (16, 256, 11008, 3)])
def test_fp16_activations_into_prepared_weights(abq, oracle, cuda, M, N, K, q):
    """ABQ_FLAG_X_HALF together with prepared weights: the codes of the FasterTransformer quantiser, the exact product."""
    rng = np.random.default_rng(M + N)
    x = rng.normal(0, 2.0, size=(M, K)).astype(np.float16)
    w = rand_codes(rng, N, K, q, False)
    qs = torch.full((1,), 13.0, dtype=torch.float32, device="cuda")
    got, _ = run_prepared(abq, torch.from_numpy(x).cuda(), planes_dev(oracle, w, q), M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False,
                          flags=abq.FLAG_X_HALF, x_quant_scale=qs)
    _, codes = oracle.quantize_half_compat(x, 13.0, 8)
    codes = ((codes + 128) % 256) - 128
    assert np.array_equal(got, oracle.gemm_values_blas(codes, w))


def test_widths_without_a_prepared_form_read_the_planes(abq, oracle, cuda):
    from abq_llm_b200 import binding as B
    M, N, K, p, q = 4, 256, 512, 8, 5
    rng = np.random.default_rng(1)
    x, w = rand_codes(rng, M, K, p, True), rand_codes(rng, N, K, q, False)
    out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    junk = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    prm = B.make_params(M, N, K, planes_dev(oracle, x, p), planes_dev(oracle, w, q), out, x_bits=p, w_bits=q, x_signed=True, w_signed=False,
                        route=abq.ROUTE_I8_MMA, flags=abq.FLAG_WEIGHTS_PREPARED, w_prepared=junk)
    assert abq.gemm_prepared_weight_bytes(prm) == 0
    st = abq.gemm_init(prm)
    abq.gemm_prepare_weights(st)  # nothing to do
    abq.gemm_exec(st)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.gemm_values_blas(x, w))


@pytest.mark.parametrize("N,K", [(4096, 4096), (12288, 4096), (11008, 4096), (4096, 11008)])
@pytest.mark.parametrize("q", [2, 3, 4])
def test_full_size_sweep_shapes(abq, oracle, cuda, N, K, q):
    """The 36 GEMMs of the benchmark at full size on prepared weights: fp16 against the oracle, int32 bit for bit, and the
    fp16 bits of the plane path where both fold the same groups in the same order (they do not promise that: only
    reported closeness is required)."""
    rng = np.random.default_rng(N + K + q)
    w = rand_codes(rng, N, K, q, False)
    ws = rng.uniform(0.001, 0.02, size=(N, K // 128)).astype(np.float16)
    wz = rng.integers(0, 1 << q, size=(N, K // 128)).astype(np.uint8)
    wp, dws, dwz = planes_dev(oracle, w, q), dev(ws), dev(wz)
    for M in (1, 4, 16):
        x = np.clip(np.rint(rng.normal(0, 30, size=(M, K))), -128, 127).astype(np.int32)
        xp = planes_dev(oracle, x, 8)
        got, _ = run_prepared(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False, out_fp16=True, scale_mode=abq.SCALE_GROUP,
                              group_size=128, w_scale=dws, w_zero=dwz, flags=abq.FLAG_PDL)
        check_close(got, oracle.dequant_gemm(x, w, ws, wz.astype(np.int32), None, 128))
        acc, _ = run_prepared(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False)
        assert np.array_equal(acc, oracle.gemm_values_blas(x, w)), f"M={M}"


def test_tuning_table_entry_is_honoured(abq, oracle, cuda, monkeypatch, tmp_path):
    """A table line for the problem changes the launch shape (here: sixteen warps, one CTA per SM, 74 CTAs) and nothing else."""
    M, N, K, q = 4, 2048, 1024, 4
    rng = np.random.default_rng(7)
    x, w = rand_codes(rng, M, K, 8, True), rand_codes(rng, N, K, q, False)
    xp, wp = planes_dev(oracle, x, 8), planes_dev(oracle, w, q)
    base, st0 = run_prepared(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False)
    # the table is read once per process: this test can only check a process that has not planned yet, so it runs a child
    import subprocess, sys, textwrap
    table = tmp_path / "table.txt"
    table.write_text(f"{q} 8 4 {N} {K} 0 0 : 0 0 0 16 1 74 0 0 0\n")
    code = textwrap.dedent(f"""
        import sys, ctypes
        sys.path.insert(0, {str(__import__('pathlib').Path(__file__).resolve().parent)!r}); sys.path.insert(0, {str(__import__('pathlib').Path(__file__).resolve().parent.parent)!r})
        from conftest import load_package
        abq = load_package()
        from abq_llm_b200 import binding as B
        p = B.GemmParams(); p.M, p.N, p.K = {M}, {N}, {K}; p.X = p.W = p.D = 4096; p.x_bits, p.w_bits, p.x_signed = 8, {q}, 1
        p.route = 2; p.flags = abq.FLAG_WEIGHTS_PREPARED; p.w_prepared = 4096
        st = B.GemmState(); assert abq.lib().abq_gemm_init(ctypes.byref(p), ctypes.byref(st)) == 0
        print(st.grid[0], st.block[0])
    """)
    env = dict(__import__("os").environ, ABQ_TUNE_TABLE=str(table))
    env.pop("ABQ_TUNE_IGNORE", None)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert out.returncode == 0, out.stderr[-1500:]
    assert out.stdout.split() == ["74", "512"], out.stdout
    assert (st0.grid[0], st0.block[0]) != (74, 512)
    assert np.array_equal(base, oracle.gemm_values_blas(x, w))


def test_tuning_table_shapes_the_plane_kernel_too(abq, oracle, cuda, tmp_path):
    """A table line with planes = 1 sends the problem to the kernel that reads the planes and may give it a launch shape: here
    K split over four CTAs and eight warps, against the heuristic's unsplit sixteen."""
    import subprocess, sys, textwrap
    M, N, K, q = 16, 512, 4096, 2
    table = tmp_path / "table.txt"
    table.write_text(f"{q} 8 16 {N} {K} 0 0 : 0 2 0 8 0 0 4 0 1\n")
    code = textwrap.dedent(f"""
        import sys, ctypes
        sys.path.insert(0, {str(__import__('pathlib').Path(__file__).resolve().parent)!r}); sys.path.insert(0, {str(__import__('pathlib').Path(__file__).resolve().parent.parent)!r})
        import torch
        from conftest import load_package
        abq = load_package()
        from abq_llm_b200 import binding as B
        buf = torch.zeros(16 << 20, dtype=torch.uint8, device="cuda")
        p = B.GemmParams(); p.M, p.N, p.K = {M}, {N}, {K}; p.X = p.W = p.D = p.workspace = buf.data_ptr(); p.workspace_bytes = 16 << 20
        p.x_bits, p.w_bits, p.x_signed = 8, {q}, 1
        p.route = 2; p.flags = abq.FLAG_WEIGHTS_PREPARED; p.w_prepared = buf.data_ptr()
        st = B.GemmState(); assert abq.lib().abq_gemm_init(ctypes.byref(p), ctypes.byref(st)) == 0
        print(abq.state_kernel(st), st.cluster, st.block[0])
    """)
    env = dict(__import__("os").environ, ABQ_TUNE_TABLE=str(table))
    env.pop("ABQ_TUNE_IGNORE", None)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-1500:]
    assert out.stdout.split() == ["decode_kernel", "4", "256"], out.stdout
    env["ABQ_TUNE_IGNORE"] = "1"
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-1500:]
    assert out.stdout.split()[0] == "stream_kernel", out.stdout


TALL_CASES = [
    # M, N, K, w_bits, group (0: int32 output, no scales)   -- 17..32 token rows go through one launch of the 32-row variant
    (17, 520, 1152, 4, 0), (32, 4096, 4096, 4, 0), (24, 200, 4096, 2, 0), (32, 1024, 11008, 3, 0), (33, 320, 1280, 8, 0), (64, 136, 2048, 2, 0),
    (40, 512, 4096, 4, 0), (17, 264, 640, 3, 128), (32, 4096, 4096, 4, 128), (32, 512, 11008, 2, 128), (25, 1000, 2048, 8, 128), (48, 320, 1536, 2, 64),
    (32, 5120, 5120, 2, 64),
]


@pytest.mark.parametrize("rows32", ["0", "1"], ids=["launches_of_16", "launches_of_32"])
@pytest.mark.parametrize("M,N,K,q,group", TALL_CASES)
def test_more_than_16_token_rows(abq, oracle, cuda, monkeypatch, M, N, K, q, group, rows32):
    """More than 16 token rows on prepared weights, as launches of 16 rows (default) and as launches of 32 rows (opt-in: one
    read of the weights per 32 rows): a ragged last launch, K ranges that must be split over CTAs, per-group scales and
    zero points, scale groups of 64."""
    monkeypatch.setenv("ABQ_STREAM_ROWS32", rows32)
    rng = np.random.default_rng(M * 17 + N + K + q + group)
    x, w = rand_codes(rng, M, K, 8, True), rand_codes(rng, N, K, q, False)
    xp, wp = planes_dev(oracle, x, 8), planes_dev(oracle, w, q)
    if not group:
        got, st = run_prepared(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False, calls=2)
        assert abq.state_kernel(st) == "stream_kernel"
        assert np.array_equal(got, oracle.gemm_values_blas(x, w))
        return
    G = K // group
    scale = rng.uniform(0.001, 0.02, size=(N, G)).astype(np.float16)
    zero = rng.integers(0, 1 << q, size=(N, G)).astype(np.uint8)
    tok = rng.uniform(0.5, 2.0, size=M).astype(np.float32)
    got, st = run_prepared(abq, xp, wp, M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False, out_fp16=True, scale_mode=abq.SCALE_GROUP,
                           group_size=group, w_scale=dev(scale), w_zero=dev(zero), x_scale=dev(tok), calls=2)
    assert abq.state_kernel(st) == "stream_kernel"
    check_close(got, oracle.dequant_gemm(x, w, scale, zero.astype(np.int32), tok, group))


def test_fp16_activations_32_rows(abq, oracle, cuda, monkeypatch):
    """ABQ_FLAG_X_HALF with 32 token rows in one launch: the record builder quantises 32 rows of fp16 activations."""
    monkeypatch.setenv("ABQ_STREAM_ROWS32", "1")
    M, N, K, q = 32, 512, 4096, 4
    rng = np.random.default_rng(321)
    x = rng.normal(0, 2.0, size=(M, K)).astype(np.float16)
    w = rand_codes(rng, N, K, q, False)
    qs = torch.full((1,), 13.0, dtype=torch.float32, device="cuda")
    got, _ = run_prepared(abq, torch.from_numpy(x).cuda(), planes_dev(oracle, w, q), M, N, K, x_bits=8, w_bits=q, x_signed=True, w_signed=False,
                          flags=abq.FLAG_X_HALF, x_quant_scale=qs)
    _, codes = oracle.quantize_half_compat(x, 13.0, 8)
    codes = ((codes + 128) % 256) - 128
    assert np.array_equal(got, oracle.gemm_values_blas(codes, w))


@pytest.mark.parametrize("M,N,K,q,group,prepared", [(1, 4096, 4096, 4, 0, True), (5, 264, 1152, 2, 128, True), (16, 512, 4096, 4, 0, True), (16, 1024, 11008, 3, 128, True),
                                                     (33, 320, 1280, 4, 0, True), (4, 520, 1024, 4, 0, False), (16, 136, 4096, 5, 128, False)])
def test_residual_added_in_the_epilogue(abq, oracle, cuda, M, N, K, q, group, prepared):
    """params.residual: D = half(result) + residual, bit for bit what the same GEMM without it followed by an fp16 add gives,
    on the prepared-weights kernel and on the kernel that reads the planes (also across launches of 16 rows and with K split
    over CTAs); the tensor-core route has no such input and says so."""
    from abq_llm_b200 import binding as B
    rng = np.random.default_rng(M + N + K + q)
    x, w = rand_codes(rng, M, K, 8, True), rand_codes(rng, N, K, q, False)
    xp, wp = planes_dev(oracle, x, 8), planes_dev(oracle, w, q)
    shape = (N, K // group) if group else (N,)
    scale = dev(rng.uniform(0.001, 0.01, size=shape).astype(np.float16))
    zero = dev(rng.integers(0, 1 << q, size=shape).astype(np.uint8))
    res = torch.randn((M, N), device="cuda").half()
    ws = torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, 8, q, abq.ROUTE_I8_MMA)), dtype=torch.uint8, device="cuda")
    outs = []
    prep = None
    for residual in (None, res):
        out = torch.zeros((M, N), dtype=torch.float16, device="cuda")
        p = B.make_params(M, N, K, xp, wp, out, x_bits=8, w_bits=q, x_signed=True, w_signed=False, out_dtype=abq.OUT_FP16,
                          scale_mode=abq.SCALE_GROUP if group else abq.SCALE_CHANNEL, group_size=group, w_scale=scale, w_zero=zero,
                          route=abq.ROUTE_I8_MMA, flags=abq.FLAG_WEIGHTS_PREPARED if prepared else 0, workspace=ws, residual=residual)
        if prepared:
            if prep is None:
                prep = torch.empty(abq.gemm_prepared_weight_bytes(p), dtype=torch.uint8, device="cuda")
            p.w_prepared = prep.data_ptr()
        st = abq.gemm_init(p)
        assert abq.state_kernel(st) == ("stream_kernel" if prepared else "decode_kernel")
        if prepared:
            abq.gemm_prepare_weights(st)
        abq.gemm_exec(st)
        torch.cuda.synchronize()
        outs.append(out)
    assert torch.equal(outs[1], outs[0] + res)  # torch's fp16 add: the exact sum rounded once, as __hadd
    big = torch.zeros((64, N), dtype=torch.float16, device="cuda")
    wsu = torch.empty(abq.gemm_workspace_bytes(64, N, K, 8, q, abq.ROUTE_I8_UMMA), dtype=torch.uint8, device="cuda")
    xb = planes_dev(oracle, rand_codes(rng, 64, K, 8, True), 8)
    with pytest.raises(abq.AbqError) as err:
        abq.gemm_init(B.make_params(64, N, K, xb, wp, big, x_bits=8, w_bits=q, x_signed=True, w_signed=False, out_dtype=abq.OUT_FP16,
                                    scale_mode=abq.SCALE_CHANNEL, w_scale=dev(np.ones(N, dtype=np.float16)), route=abq.ROUTE_I8_UMMA, workspace=wsu,
                                    residual=big))
    assert err.value.status == 2  # ABQ_ERR_UNSUPPORTED
