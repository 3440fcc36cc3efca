"""The C++ side of the drop-in boundary, compiled and run: a caller written against the reference's launch interface
(named Init/Exec pairs, launchWmmaAnyKernel, class ABQGEMMWrapper) builds against include/abq_compat.hpp and the shared
library unchanged and gives the oracle's results bit for bit.  Also the Python mirror of the wrapper class.

The wrapper cases hand over the workspace FasterTransformer's layers allocate (the activation planes only,
layers/FfnLayer.cc:670-673), so for more than 16 tokens the call runs on the library's built-in scratch array; scale_out
is a float whose first two bytes are read as fp16, as abq_gemm_wrapper.cu:125-126 does."""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import rand_codes

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "compat" / "compat_driver.cpp"
EXE = ROOT / "tests" / "_build" / "compat_driver"


def build_driver(abq) -> Path:
    lib = abq.lib_path()
    deps = [SRC, ROOT / "include" / "abq_compat.hpp", ROOT / "include" / "abq_b200.h"]
    if not EXE.exists() or any(d.stat().st_mtime > EXE.stat().st_mtime for d in deps):
        EXE.parent.mkdir(exist_ok=True)
        cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
        subprocess.run(["g++", "-std=c++17", "-O1", f"-I{cuda / 'include'}", f"-I{ROOT / 'include'}", str(SRC), "-o", str(EXE),
                        f"-L{lib.parent}", "-labq_b200", f"-L{cuda / 'lib64'}", "-lcudart", f"-Wl,-rpath,{lib.parent}"], check=True)
    return EXE


def run_driver(abq, what, tmp_path, M, N, K, files):
    for name, arr in files.items():
        np.ascontiguousarray(arr).tofile(tmp_path / name)
    res = subprocess.run([str(build_driver(abq)), what, str(tmp_path), str(M), str(N), str(K)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, f"exit {res.returncode}: {res.stdout[-1000:]} {res.stderr[-1000:]}"
    assert "[ABQ][Error]" not in res.stdout, res.stdout
    return res


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (8, 1000, 1152), (48, 512, 1024)])
def test_named_init_exec_pairs(abq, oracle, cuda, tmp_path, M, N, K):
    """ABQ_COMPAT_DEFINE_CONFIG pairs with the names FasterTransformer uses for W2A8; no workspace installed, so more than 16
    rows run on the built-in scratch array."""
    rng = np.random.default_rng(M + N)
    x, w = rand_codes(rng, M, K, 8, True), rand_codes(rng, N, K, 2, True)
    res = run_driver(abq, "initexec", tmp_path, M, N, K, {"x.bin": oracle.pack(x, 8), "w.bin": oracle.pack(w, 2)})
    assert "AqBMMAInitFn" in res.stderr  # the refused bias is reported, not ignored
    got = np.fromfile(tmp_path / "d.bin", dtype=np.int32).reshape(M, N)
    assert np.array_equal(got, oracle.gemm_values_blas(x, w))


@pytest.mark.parametrize("M,N,K", [(128, 4096, 4096), (16, 256, 512), (5, 48, 128)])
def test_launch_wmma_any_kernel(abq, oracle, cuda, tmp_path, M, N, K):
    """launchWmmaAnyKernel<QuantType<4, 4, false>, ...> with the tile arguments of engine/test_w4a4_uint_wmma.cu:230."""
    rng = np.random.default_rng(M * 7 + N)
    x, w = rand_codes(rng, M, K, 4, False), rand_codes(rng, N, K, 4, False)
    run_driver(abq, "wmma_any", tmp_path, M, N, K, {"x.bin": oracle.pack(x, 4), "w.bin": oracle.pack(w, 4)})
    got = np.fromfile(tmp_path / "d.bin", dtype=np.int32).reshape(M, N)
    want = oracle.gemm_values_blas(x, w)
    assert np.array_equal(got, want)
    if M * N * K <= 1 << 22:
        assert np.array_equal(want, oracle.compute_ref(oracle.pack(w, 4), oracle.pack(x, 4), False, False))


def _wrapper_inputs(rng, M, N, K):
    x = rng.normal(0, 2.0, size=(M, K)).astype(np.float16)
    w = rand_codes(rng, N, K, 2, True)
    scale = np.array([11.5], dtype=np.float32)
    out_scale = np.float16(0.0123)
    scale_out = np.zeros(1, dtype=np.float32)
    scale_out.view(np.uint16)[0] = out_scale.view(np.uint16)   # the low two bytes of the float hold the fp16 scale
    scale_out.view(np.uint16)[1] = 0x7777                      # the rest must be ignored
    return x, w, scale, out_scale, scale_out


def _wrapper_expected(oracle, x, w, scale, out_scale, signed):
    planes, codes = oracle.quantize_half_compat(x, float(scale[0]), 8)
    vals = ((codes + 128) % 256) - 128 if signed else codes % 256
    wv = w if signed else w % 4
    return planes, oracle.dequant_tensor_compat(oracle.gemm_values_blas(vals, wv), out_scale)


@pytest.mark.parametrize("what", ["wrapper", "wrapper_u", "wrapper_p"])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (7, 640, 1152), (40, 768, 2048)])
def test_ft_wrapper_class(abq, oracle, cuda, tmp_path, what, M, N, K):
    rng = np.random.default_rng(M + K)
    x, w, scale, out_scale, scale_out = _wrapper_inputs(rng, M, N, K)
    signed = what != "wrapper_u"
    run_driver(abq, what, tmp_path, M, N, K, {"x.bin": x, "w.bin": oracle.pack(w, 2), "scale.bin": scale, "scale_out.bin": scale_out})
    planes, want = _wrapper_expected(oracle, x, w, scale, out_scale, signed)
    got = np.fromfile(tmp_path / "d.bin", dtype=np.float16).reshape(M, N)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    if not signed:
        assert np.array_equal(np.fromfile(tmp_path / "planes.bin", dtype=np.uint32).reshape(planes.shape), planes)


@pytest.mark.parametrize("signed", [True, False])
@pytest.mark.parametrize("M,N,K", [(1, 1024, 4096), (40, 768, 2048)])
def test_python_wrapper_mirror(abq, oracle, cuda, signed, M, N, K):
    """abq_llm_b200.ABQGEMMWrapper.gemm: same argument meaning as the C++ class; its own workspace_bytes() as the size."""
    rng = np.random.default_rng(N + K)
    x, w, scale, out_scale, scale_out = _wrapper_inputs(rng, M, N, K)
    wrapper = abq.ABQGEMMWrapper(8, 2, signed)
    ws_bytes = wrapper.workspace_bytes(M, N, K)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    D = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    wp = torch.from_numpy(oracle.pack(w, 2).view(np.int32)).cuda()
    wrapper.gemm(M, N, K, torch.from_numpy(x).cuda(), wp, None, D, torch.from_numpy(scale).cuda(), None, torch.from_numpy(scale_out).cuda(),
                 False, ws, ws_bytes)
    torch.cuda.synchronize()
    _, want = _wrapper_expected(oracle, x, w, scale, out_scale, signed)
    assert np.array_equal(D.cpu().numpy().view(np.uint16), want.view(np.uint16))
    with pytest.raises(abq.AbqError):
        wrapper.gemm(M, N, K, torch.from_numpy(x).cuda(), wp, None, D, torch.from_numpy(scale).cuda(), None, torch.from_numpy(scale_out).cuda(),
                     False, ws, 16)   # the reference never checks ws_bytes; the mirror does
    with pytest.raises(abq.AbqError):
        wrapper.gemm(M, N, 100, torch.from_numpy(x).cuda(), wp, None, D, torch.from_numpy(scale).cuda(), None, torch.from_numpy(scale_out).cuda(),
                     False, ws, ws_bytes)  # "[ABQ][Error] unsupport K"
