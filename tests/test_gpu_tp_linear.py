"""The tensor-parallel block linears with the product backend on one GPU against the numpy stand-in (CPU oracle)."""
import numpy as np
import pytest
import torch

from test_tp_linear_gloo import NumpyBackend, _tp, _weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("group", [128, 0])
@pytest.mark.parametrize("M", [1, 5, 20])
def test_block_linears_match_the_oracle_backend(abq, oracle, cuda, group, M):
    tp = _tp()
    hidden, ffn, q = 256, 640, 4
    weights = _weights(tp, hidden, ffn, q, group)
    x = np.random.default_rng(M).normal(0, 1.0, size=(M, hidden)).astype(np.float16)
    want = tp.TensorParallelBlockLinears(NumpyBackend(group), hidden, ffn, 0, 1, weights, q, group).forward(x)
    dev_w = [(torch.from_numpy(c).cuda(), torch.from_numpy(s).cuda(), torch.from_numpy(z).cuda()) for c, s, z in weights]
    block = tp.TensorParallelBlockLinears(tp.AbqBackend(abq, torch), hidden, ffn, 0, 1, dev_w, q, group)
    got = block.forward(torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    got = got.cpu().numpy().astype(np.float64)
    ref = want.astype(np.float64)
    # two chained GEMMs with fp16 intermediates: a rounding difference of one intermediate moves a quantised code
    err = np.abs(got - ref)
    assert np.all(err <= 2.0 ** -6 * np.abs(ref) + 2.0 ** -7 * np.abs(ref).max()), f"max abs err {err.max():.4g} of {np.abs(ref).max():.4g}"


@pytest.mark.parametrize("M,F", [(1, 11008), (8, 5504), (32, 1376), (5, 64)])
def test_glue_kernels_match_torch(abq, cuda, M, F):
    """The library's SiLU(gate) * up and residual-add launches against the torch elementwise kernels they replace in the block
    (fp16; the SiLU uses the fast exponential: at most one fp16 step off before the product)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(M + F)
    gu = (torch.randn((M, 2 * F), device="cuda", generator=g) * 2).half()
    out = torch.empty((M, F), dtype=torch.float16, device="cuda")
    abq.swiglu_half(gu, out, M, F)
    want = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    torch.cuda.synchronize()
    err = (out.float() - want.float()).abs()
    assert bool((err <= 2.0 ** -9 * want.float().abs() + 1e-4).all()), float(err.max())
    a, b = gu[:, :F].contiguous(), gu[:, F:].contiguous()
    s = torch.empty_like(a)
    abq.add_half(a, b, s, a.numel())
    torch.cuda.synchronize()
    assert torch.equal(s, a + b)
    with pytest.raises(abq.AbqError):
        abq.swiglu_half(gu, out, M, F + 4)
