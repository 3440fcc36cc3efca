"""Pack / quantise / unpack kernels against the CPU oracle and the reference's own GPU pack kernel."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import dev, rand_codes

pytestmark = pytest.mark.gpu

SHAPES = [(1, 128), (1, 4096), (3, 384), (8, 1024), (16, 11008), (37, 640), (128, 4096)]


@pytest.mark.parametrize("rows,K", SHAPES)
@pytest.mark.parametrize("bits,signed", [(2, False), (3, True), (4, False), (8, True), (1, False), (5, False), (8, False)])
def test_pack_int32(abq, oracle, cuda, rows, K, bits, signed):
    rng = np.random.default_rng(rows * 131 + K + bits)
    codes = rand_codes(rng, rows, K, bits, signed)
    planes = torch.full((bits, rows, K // 32), 0x55, dtype=torch.int32, device="cuda")
    abq.pack_int32(dev(codes), planes, rows, K, bits)
    torch.cuda.synchronize()
    want = oracle.pack(codes, bits)
    assert np.array_equal(planes.cpu().numpy().view(np.uint32), want)


@pytest.mark.parametrize("rows,K", [(1, 128), (8, 4096), (33, 256)])
def test_pack_matches_reference_kernel(abq, oracle, cuda, rows, K):
    """The reference's own `launch_pack` (compiled from its sources) on the same device input."""
    if not oracle.ref_available():
        pytest.skip("oracle/_ref was not built")
    bits = 4
    rng = np.random.default_rng(7)
    codes = dev(rand_codes(rng, rows, K, bits, False))
    mine = torch.zeros((bits, rows, K // 32), dtype=torch.int32, device="cuda")
    theirs = torch.zeros_like(mine)
    abq.pack_int32(codes, mine, rows, K, bits)
    err = oracle.ref().launch_pack(codes.data_ptr(), theirs.data_ptr(), rows, K, bits, None)
    torch.cuda.synchronize()
    assert err == 0
    assert torch.equal(mine, theirs)


@pytest.mark.parametrize("rows,K", [(1, 128), (5, 512), (64, 4096)])
@pytest.mark.parametrize("bits", [4, 2])
def test_pack_int4(abq, oracle, cuda, rows, K, bits):
    rng = np.random.default_rng(rows + K)
    words = rng.integers(0, 1 << 32, size=rows * K // 8, dtype=np.uint64).astype(np.uint32)
    planes = torch.zeros((bits, rows, K // 32), dtype=torch.int32, device="cuda")
    abq.pack_int4(dev(words.view(np.int32)), planes, rows, K, bits)
    torch.cuda.synchronize()
    want = oracle.pack4(words, rows, K, bits)
    assert np.array_equal(planes.cpu().numpy().view(np.uint32), want)
    if oracle.ref_available() and bits == 4:
        theirs = torch.zeros_like(planes)
        assert oracle.ref().launch_pack4(dev(words.view(np.int32)).data_ptr(), theirs.data_ptr(), rows, K, bits, None) == 0
        torch.cuda.synchronize()
        assert torch.equal(planes, theirs)


@pytest.mark.parametrize("rows,K", [(1, 4096), (4, 128), (16, 11008), (50, 1024)])
@pytest.mark.parametrize("bits", [8, 4, 6])
def test_quantize_pack_half_compat(abq, oracle, cuda, rows, K, bits):
    """int(half(x) * half(scale)) truncating and unclamped, as the FasterTransformer wrapper."""
    rng = np.random.default_rng(rows * K + bits)
    x = (rng.standard_normal((rows, K)) * 2.0).astype(np.float16)
    scale = 11.37
    planes = torch.zeros((bits, rows, K // 32), dtype=torch.int32, device="cuda")
    abq.quantize_pack_half(dev(x), dev(np.array([scale], dtype=np.float32)), planes, rows, K, bits, 0)
    torch.cuda.synchronize()
    want, _ = oracle.quantize_half_compat(x, scale, bits)
    assert np.array_equal(planes.cpu().numpy().view(np.uint32), want)


@pytest.mark.parametrize("rows,K", [(1, 4096), (7, 384), (16, 11008)])
@pytest.mark.parametrize("bits", [8, 4, 2])
def test_quantize_pack_half_rtn(abq, oracle, cuda, rows, K, bits):
    rng = np.random.default_rng(rows * K + bits + 1)
    x = (rng.standard_normal((rows, K)) * 3.0).astype(np.float16)
    qmax = (1 << (bits - 1)) - 1
    row_scale = (np.abs(x.astype(np.float32)).max(axis=1) / max(qmax, 1)).astype(np.float32) * 0.3  # a third of the range is clamped
    planes = torch.zeros((bits, rows, K // 32), dtype=torch.int32, device="cuda")
    abq.quantize_pack_half(dev(x), dev(row_scale), planes, rows, K, bits, 1)
    torch.cuda.synchronize()
    want, codes = oracle.quantize_half_rtn(x, row_scale, bits)
    assert codes.min() == -(1 << (bits - 1)) and codes.max() == qmax
    assert np.array_equal(planes.cpu().numpy().view(np.uint32), want)


@pytest.mark.parametrize("rows,K", [(1, 128), (9, 1152), (64, 4096)])
@pytest.mark.parametrize("bits,signed", [(2, False), (2, True), (4, True), (7, False), (8, True), (8, False), (3, True)])
def test_unpack_int8(abq, oracle, cuda, rows, K, bits, signed):
    rng = np.random.default_rng(rows + K + bits)
    codes = rand_codes(rng, rows, K, bits, signed)
    planes = dev(oracle.pack(codes, bits).view(np.int32))
    out = torch.zeros((rows, K), dtype=torch.uint8 if (bits == 8 and not signed) else torch.int8, device="cuda")
    abq.unpack_int8(planes, out, rows, K, bits, signed)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().astype(np.int32), codes)
    assert np.array_equal(oracle.unpack(oracle.pack(codes, bits), signed), codes)
