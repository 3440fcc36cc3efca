"""Every GPU route on the golden fixtures (inputs and int32 outputs produced by the reference's own code)."""
from pathlib import Path

import numpy as np
import pytest

from helpers import dev, run_gemm

pytestmark = pytest.mark.gpu
GOLDEN = sorted(Path(__file__).resolve().parent.glob("golden/*.npz"))


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
@pytest.mark.parametrize("route", ["i8_mma", "b1_mma", "i8_umma"])
def test_routes_reproduce_reference_output(abq, cuda, path, route):
    g = np.load(path)
    M, N, K, p, q, signed, _ = (int(v) for v in g["meta"])
    rid = {"i8_mma": abq.ROUTE_I8_MMA, "b1_mma": abq.ROUTE_B1_MMA, "i8_umma": abq.ROUTE_I8_UMMA}[route]
    got, _ = run_gemm(abq, dev(g["x_planes"].view(np.int32)), dev(g["w_planes"].view(np.int32)), M, N, K, x_bits=p, w_bits=q,
                      x_signed=bool(signed), w_signed=bool(signed), route=rid)
    assert np.array_equal(got, g["d"])


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_pack_kernel_reproduces_reference_planes(abq, cuda, path):
    import torch
    g = np.load(path)
    M, N, K, p, q, _, _ = (int(v) for v in g["meta"])
    for codes, bits, want in ((g["x"], p, g["x_planes"]), (g["w"], q, g["w_planes"])):
        rows = codes.shape[0]
        planes = torch.zeros((bits, rows, K // 32), dtype=torch.int32, device="cuda")
        abq.pack_int32(dev(codes.astype(np.int32)), planes, rows, K, bits)
        torch.cuda.synchronize()
        assert np.array_equal(planes.cpu().numpy().view(np.uint32), want)
