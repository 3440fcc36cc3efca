"""abq_gemm_static_scratch: the GEMM for callers that cannot hand over (or allocate) scratch memory.

A FasterTransformer linear layer gives the GEMM wrapper a workspace that only holds the activation planes, and a
forward pass must not call cudaMalloc (device-wide synchronisation, illegal during graph capture).  This entry point
therefore runs on a scratch array built into the library.  The test drives it through the C ABI, twice in a row on the
shared array with different operands, and requires the output of the ordinary entry point (caller-owned workspace):
bit for bit for int32, and identical fp16 bits for the fused epilogue, since both run the same kernels.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import dev, planes_dev, rand_codes

pytestmark = pytest.mark.gpu


def _params(abq, M, N, K, xp, wp, out, *, p, q, signed, ws=None, fp16=False, w_scale=None):
    from abq_llm_b200 import binding as B
    return B.make_params(M, N, K, xp, wp, out, x_bits=p, w_bits=q, x_signed=signed, w_signed=signed,
                         out_dtype=abq.OUT_FP16 if fp16 else abq.OUT_INT32, scale_mode=abq.SCALE_CHANNEL if fp16 else abq.SCALE_NONE,
                         w_scale=w_scale, workspace=ws)


@pytest.mark.parametrize("fp16", [False, True])
def test_static_scratch_matches_workspace_entry_point(abq, oracle, cuda, fp16):
    M, N, K, p, q = 192, 640, 1024, 8, 4  # M > 16: the route that needs scratch (expanded int8 operands)
    assert abq.gemm_workspace_bytes(M, N, K, p, q) <= abq.STATIC_SCRATCH_BYTES
    rng = np.random.default_rng(11)
    for call in range(2):  # second call reuses the array with other data: nothing may leak from the first
        signed = call == 1
        x, w = rand_codes(rng, M, K, p, signed), rand_codes(rng, N, K, q, signed)
        xp, wp = planes_dev(oracle, x, p), planes_dev(oracle, w, q)
        scale = dev(rng.uniform(0.001, 0.02, size=N).astype(np.float16)) if fp16 else None
        dtype = torch.float16 if fp16 else torch.int32
        ref_out = torch.zeros((M, N), dtype=dtype, device="cuda")
        new_out = torch.zeros((M, N), dtype=dtype, device="cuda")
        ws = torch.empty(abq.gemm_workspace_bytes(M, N, K, p, q), dtype=torch.uint8, device="cuda")
        abq.gemm(_params(abq, M, N, K, xp, wp, ref_out, p=p, q=q, signed=signed, ws=ws, fp16=fp16, w_scale=scale))
        abq.gemm_static_scratch(_params(abq, M, N, K, xp, wp, new_out, p=p, q=q, signed=signed, fp16=fp16, w_scale=scale))
        torch.cuda.synchronize()
        assert torch.equal(ref_out.view(torch.int16) if fp16 else ref_out, new_out.view(torch.int16) if fp16 else new_out)
        if not fp16:
            assert np.array_equal(new_out.cpu().numpy(), oracle.gemm_values_blas(x, w))


def test_static_scratch_rejects_oversized_problem(abq, cuda):
    M, N, K = 4096, 4096, 4096  # needs 32 MiB of scratch, the array holds 16 MiB
    assert abq.gemm_workspace_bytes(M, N, K, 8, 8) > abq.STATIC_SCRATCH_BYTES
    from abq_llm_b200 import binding as B
    one = torch.zeros(256, dtype=torch.int32, device="cuda")
    p = B.make_params(M, N, K, one, one, one, x_bits=8, w_bits=8, x_signed=True, w_signed=True)
    with pytest.raises(abq.AbqError) as err:
        abq.gemm_static_scratch(p)
    assert err.value.status == 3  # ABQ_ERR_WORKSPACE, before anything is launched


def test_static_scratch_decode_split_k_twice_in_a_row(abq, oracle, cuda):
    """16 tokens with K = 11008: the decode route splits K over CTAs and keeps its arrival counters and partial sums at
    the head of the scratch -- here the shared array, which the previous test left full of other data.  Two calls in a
    row with different operands must both match the entry point with a caller-owned workspace and the oracle."""
    M, N, K, p, q = 16, 1024, 11008, 8, 4
    rng = np.random.default_rng(23)
    for call in range(2):
        x, w = rand_codes(rng, M, K, p, True), rand_codes(rng, N, K, q, False)
        xp, wp = planes_dev(oracle, x, p), planes_dev(oracle, w, q)
        ref_out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
        new_out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
        ws = torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, p, q)), dtype=torch.uint8, device="cuda")
        from abq_llm_b200 import binding as B
        kw = dict(x_bits=p, w_bits=q, x_signed=True, w_signed=False, route=abq.ROUTE_I8_MMA)
        abq.gemm(B.make_params(M, N, K, xp, wp, ref_out, workspace=ws, **kw))
        abq.gemm_static_scratch(B.make_params(M, N, K, xp, wp, new_out, **kw))
        torch.cuda.synchronize()
        assert torch.equal(ref_out, new_out)
        assert np.array_equal(new_out.cpu().numpy(), oracle.gemm_values_blas(x, w))


def test_static_scratch_refuses_prepared_weights(abq, cuda):
    """Prepared weights are a copy that lives in the caller's own workspace; on the shared array the "copy" would be
    whatever the last call left there, so the flag is an argument error and nothing is launched."""
    from abq_llm_b200 import binding as B
    one = torch.zeros(4096, dtype=torch.int32, device="cuda")
    p = B.make_params(64, 64, 128, one, one, one, x_bits=4, w_bits=4, x_signed=False, w_signed=False, flags=abq.FLAG_WEIGHTS_PREPARED)
    with pytest.raises(abq.AbqError) as err:
        abq.gemm_static_scratch(p)
    assert err.value.status == 1  # ABQ_ERR_INVALID_ARG


def test_static_scratch_serves_decode_route_with_callers_prepared_copy(abq, oracle, cuda):
    """The one prepared-weights combination the shared array can serve: the decode route with the prepared copy in the
    caller's own w_prepared buffer (the scratch then only holds split-K partial sums, here 16 tokens with K = 11008)."""
    from abq_llm_b200 import binding as B
    M, N, K, p, q = 16, 512, 11008, 8, 4
    rng = np.random.default_rng(29)
    x, w = rand_codes(rng, M, K, p, True), rand_codes(rng, N, K, q, False)
    xp, wp = planes_dev(oracle, x, p), planes_dev(oracle, w, q)
    out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    ws = torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, p, q, abq.ROUTE_I8_MMA)), dtype=torch.uint8, device="cuda")
    kw = dict(x_bits=p, w_bits=q, x_signed=True, w_signed=False, route=abq.ROUTE_I8_MMA, flags=abq.FLAG_WEIGHTS_PREPARED)
    nbytes = abq.gemm_prepared_weight_bytes(B.make_params(M, N, K, xp, wp, out, **kw))
    assert nbytes > 0
    prep = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    abq.gemm_prepare_weights(abq.gemm_init(B.make_params(M, N, K, xp, wp, out, workspace=ws, w_prepared=prep, **kw)))
    torch.cuda.synchronize()
    for _ in range(2):
        out.fill_(-1)
        abq.gemm_static_scratch(B.make_params(M, N, K, xp, wp, out, w_prepared=prep, **kw))
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), oracle.gemm_values_blas(x, w))
