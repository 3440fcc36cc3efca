"""(Residual add ->) RMSNorm -> quantiser -> planes in one launch (abq_rmsnorm_quantize_pack_half).

The kernel's fp16 intermediates are outputs too, so every stage is pinned separately: the sum is the fp16 add bit for bit;
the normalised row is within one fp16 unit in the last place of the float64 formula (the kernel works in fp32 and rounds
once); the planes are EXACTLY the oracle's quantiser (the FasterTransformer one, or round-to-nearest with per-token
scales) applied to the normalised row the kernel wrote, i.e. what the separate normalisation and pack kernels of the
reference's FasterTransformer fork would have produced from it."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ulp16(a):
    a = np.abs(a.astype(np.float64))
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -14)))
    return 2.0 ** (e - 10)


@pytest.mark.parametrize("rows,K,bits,mode,residual", [(1, 4096, 8, 0, False), (5, 11008, 8, 0, True), (16, 5120, 4, 1, True), (3, 128, 8, 2, False),
                                                      (33, 4096, 8, 2, True), (2, 16384, 6, 2, False), (7, 1152, 2, 1, False)])
def test_rmsnorm_quantize_pack(abq, oracle, cuda, rows, K, bits, mode, residual):
    rng = np.random.default_rng(rows * 31 + K + bits)
    a = rng.normal(0, 1.0, size=(rows, K)).astype(np.float16)
    b = rng.normal(0, 0.5, size=(rows, K)).astype(np.float16) if residual else None
    gamma = rng.uniform(0.5, 1.5, size=K).astype(np.float16)
    eps = 1e-6
    da, dg = torch.from_numpy(a).cuda(), torch.from_numpy(gamma).cuda()
    db = torch.from_numpy(b).cuda() if residual else None
    sum_out = torch.zeros((rows, K), dtype=torch.float16, device="cuda") if residual else None
    y_out = torch.zeros((rows, K), dtype=torch.float16, device="cuda")
    planes = torch.zeros((bits, rows, K // 32), dtype=torch.int32, device="cuda")
    qmax = (1 << (bits - 1)) - 1
    scale_np = {0: np.array([9.0], dtype=np.float32), 1: rng.uniform(0.01, 0.05, size=rows).astype(np.float32), 2: None}[mode]
    scale = None if scale_np is None else torch.from_numpy(scale_np).cuda()
    row_scale = torch.zeros(rows, dtype=torch.float32, device="cuda") if mode == 2 else None
    abq.rmsnorm_quantize_pack_half(da, dg, eps, rows, K, bits, mode, residual=db, sum_out=sum_out, scale=scale, row_scale_out=row_scale,
                                   planes=planes, y_out=y_out)
    torch.cuda.synchronize()
    s = a
    if residual:
        s = (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16)  # the fp16 add: exact sum, one rounding
        assert np.array_equal(sum_out.cpu().numpy().view(np.uint16), s.view(np.uint16))
    s64 = s.astype(np.float64)
    want = s64 / np.sqrt(np.mean(s64 * s64, axis=1, keepdims=True) + eps) * gamma.astype(np.float64)
    y = y_out.cpu().numpy()
    assert np.all(np.abs(y.astype(np.float64) - want) <= _ulp16(want)), "normalised row off by more than one fp16 ulp"
    if mode == 0:
        want_planes, _ = oracle.quantize_half_compat(y, 9.0, bits)
    else:
        if mode == 2:
            rs = (np.abs(y).max(axis=1).astype(np.float32) / np.float32(qmax)).astype(np.float32)
            assert np.array_equal(row_scale.cpu().numpy(), rs)
        else:
            rs = scale_np
        want_planes, _ = oracle.quantize_half_rtn(y, rs, bits)
    assert np.array_equal(planes.cpu().numpy().view(np.uint32), want_planes)


def test_rmsnorm_only_and_argument_checks(abq, cuda):
    rows, K = 4, 4096
    x = torch.randn((rows, K), dtype=torch.float16, device="cuda")
    g = torch.ones(K, dtype=torch.float16, device="cuda")
    y = torch.zeros_like(x)
    abq.rmsnorm_quantize_pack_half(x, g, 1e-5, rows, K, 8, 0, y_out=y)  # no planes: normalisation only
    torch.cuda.synchronize()
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(dim=1, keepdim=True) + 1e-5)
    assert torch.allclose(y.float(), ref, rtol=2e-3, atol=1e-4)
    with pytest.raises(abq.AbqError):
        abq.rmsnorm_quantize_pack_half(x, g, 1e-5, rows, K, 8, 0)                       # nothing to write
    with pytest.raises(abq.AbqError):
        abq.rmsnorm_quantize_pack_half(x, g, 1e-5, rows, 32768, 8, 0, y_out=y)          # K beyond what a CTA holds
    with pytest.raises(abq.AbqError):
        abq.rmsnorm_quantize_pack_half(x, g, 1e-5, rows, K, 8, 0, planes=y)             # mode 0 needs its scale
