"""ABQ_FLAG_X_HALF: fp16 activations quantised inside the GEMM call.  The result must equal, bit for bit, the two-step
path it replaces (abq_quantize_pack_half mode 0, then the GEMM on the planes) on both int8 routes."""
import numpy as np
import pytest
import torch

from helpers import dev, planes_dev, rand_codes

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,p,q,mode", [(1, 4096, 4096, 8, 2, "group"), (5, 320, 1152, 8, 4, "int32"), (16, 512, 11008, 8, 3, "group"),
                                            (3, 128, 640, 4, 4, "channel"), (40, 256, 1024, 8, 4, "group"), (300, 1000, 1152, 8, 3, "int32"),
                                            (512, 4096, 4096, 4, 4, "channel")])
def test_fused_quantisation_equals_pack_then_gemm(abq, oracle, cuda, M, N, K, p, q, mode):
    from abq_llm_b200 import binding as B
    rng = np.random.default_rng(M + N + K)
    x = torch.from_numpy(rng.normal(0, 2.0, size=(M, K)).astype(np.float16)).cuda()
    qs = torch.full((1,), 13.0 if p == 8 else 1.5, dtype=torch.float32, device="cuda")
    w = rand_codes(rng, N, K, q, False)
    wp = planes_dev(oracle, w, q)
    kw = dict(x_bits=p, w_bits=q, x_signed=True, w_signed=False)
    if mode == "group":
        kw.update(out_dtype=abq.OUT_FP16, scale_mode=abq.SCALE_GROUP, group_size=128,
                  w_scale=dev(rng.uniform(0.001, 0.02, size=(N, K // 128)).astype(np.float16)),
                  w_zero=dev(rng.integers(0, 1 << q, size=(N, K // 128)).astype(np.uint8)))
    elif mode == "channel":
        kw.update(out_dtype=abq.OUT_FP16, scale_mode=abq.SCALE_CHANNEL, w_scale=dev(rng.uniform(0.001, 0.02, size=N).astype(np.float16)),
                  w_zero=dev(rng.integers(0, 1 << q, size=N).astype(np.uint8)))
    dtype = torch.int32 if mode == "int32" else torch.float16
    ws = torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, p, q)), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # two steps
    planes = torch.empty((p, M, K // 32), dtype=torch.int32, device="cuda")
    abq.quantize_pack_half(x, qs, planes, M, K, p, 0)
    want = torch.full((M, N), -1, dtype=dtype, device="cuda")
    abq.gemm_exec(abq.gemm_init(B.make_params(M, N, K, planes, wp, want, workspace=ws, status_word=status, **kw)))
    torch.cuda.synchronize()
    # one call
    got = torch.full((M, N), -2, dtype=dtype, device="cuda")
    st = abq.gemm_init(B.make_params(M, N, K, x, wp, got, workspace=ws, status_word=status, flags=abq.FLAG_X_HALF, x_quant_scale=qs, **kw))
    abq.gemm_exec(st)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(got, want), f"{int((got != want).sum())} of {got.numel()} differ (route {st.route})"
    # and the codes are what the oracle's restatement of the quantiser gives
    if mode == "int32":
        _, codes = oracle.quantize_half_compat(x.cpu().numpy(), float(qs.item()), p)
        half = 1 << (p - 1)
        codes = ((codes + half) % (2 * half)) - half
        assert np.array_equal(got.cpu().numpy(), oracle.gemm_values_blas(codes, w))


def test_rejected_combinations(abq, cuda):
    from abq_llm_b200 import binding as B
    x = torch.zeros((1, 128), dtype=torch.float16, device="cuda")
    w = torch.zeros((2, 16, 4), dtype=torch.int32, device="cuda")
    out = torch.zeros((1, 16), dtype=torch.int32, device="cuda")
    with pytest.raises(abq.AbqError):   # no scale
        abq.gemm_init(B.make_params(1, 16, 128, x, w, out, x_bits=8, w_bits=2, x_signed=True, w_signed=False, flags=abq.FLAG_X_HALF))
    qs = torch.ones(1, device="cuda")
    with pytest.raises(abq.AbqError):   # unsigned activations
        abq.gemm_init(B.make_params(1, 16, 128, x, w, out, x_bits=8, w_bits=2, x_signed=False, w_signed=False, flags=abq.FLAG_X_HALF,
                                    x_quant_scale=qs))
    with pytest.raises(abq.AbqError):   # the 1-bit route needs planes
        abq.gemm_init(B.make_params(1, 16, 128, x, w, out, x_bits=8, w_bits=2, x_signed=True, w_signed=False, flags=abq.FLAG_X_HALF,
                                    x_quant_scale=qs, route=abq.ROUTE_B1_MMA))
