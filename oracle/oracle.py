"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Loads ``oracle/_build/libabq_oracle.so`` (built from ``abq_oracle.c`` by ``oracle/Makefile``) and,
when present, ``oracle/_ref/libabq_ref.so`` (the reference's own ``compute_ref`` / ``init_matrix``
/ ``launch_pack`` compiled from the reference sources).  Nothing in the product imports this
module; it exists for the tests, the smoke check and the benchmark's CPU-baseline leg.

Reference citations are given per function in ``abq_oracle.c``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libabq_oracle.so"
_REF_PATH = _HERE / "_ref" / "libabq_ref.so"
_REF_GPU_PATH = _HERE / "_ref" / "libabq_ref_gpu.so"
_REF_SAMPLED_PATH = _HERE / "_ref" / "libabq_ref_gpu_sampled.so"

_i32p = ctypes.POINTER(ctypes.c_int32)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def build(force: bool = False) -> None:
    """Compile the C restatement (and the reference library when its sources are mounted)."""
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < (_HERE / "abq_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "all"], check=True, capture_output=True)
    # the reference checkout: ABQ_REFERENCE_ROOT, else a directory named "reference" beside this repository
    ref_root = os.environ.get("ABQ_REFERENCE_ROOT", str(_HERE.parent.parent / "reference"))
    if os.path.isdir(os.path.join(ref_root, "engine")) and (force or not _REF_PATH.exists()):
        subprocess.run(["make", "-C", str(_HERE), "ref", f"REF={ref_root}"], check=True, capture_output=True)
    if os.path.isdir(os.path.join(ref_root, "engine")) and (force or not _REF_GPU_PATH.exists()):
        subprocess.run(["make", "-C", str(_HERE), "refgpu", f"REF={ref_root}"], check=True, capture_output=True)
    if os.path.isdir(os.path.join(ref_root, "engine")) and (force or not _REF_SAMPLED_PATH.exists()):
        subprocess.run(["make", "-C", str(_HERE), "refsampled", f"REF={ref_root}"], check=True, capture_output=True)


_lib = None
_ref = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        L = ctypes.CDLL(str(_LIB_PATH))
        L.abq_oracle_threads.restype = ctypes.c_int
        L.abq_oracle_set_threads.argtypes = [ctypes.c_int]
        L.abq_oracle_srand.argtypes = [ctypes.c_uint]
        L.abq_oracle_init_matrix.argtypes = [_i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.abq_oracle_pack.argtypes = [_i32p, _u32p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.abq_oracle_pack4.argtypes = [_u32p, _u32p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.abq_oracle_compute_ref.argtypes = [_u32p, _u32p, _i32p] + [ctypes.c_int] * 9
        L.abq_oracle_unpack.argtypes = [_u32p, _i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.abq_oracle_gemm_values.argtypes = [_i32p, _i32p, _i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.abq_oracle_half_to_float.argtypes = [ctypes.c_uint16]
        L.abq_oracle_half_to_float.restype = ctypes.c_float
        L.abq_oracle_float_to_half.argtypes = [ctypes.c_float]
        L.abq_oracle_float_to_half.restype = ctypes.c_uint16
        L.abq_oracle_quantize_half_compat.argtypes = [_u16p, ctypes.c_float, _u32p, _i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.abq_oracle_quantize_half_rtn.argtypes = [_u16p, _f32p, _u32p, _i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.abq_oracle_dequant_tensor_compat.argtypes = [_i32p, ctypes.c_uint16, _u16p, ctypes.c_long]
        L.abq_oracle_dequant_gemm.argtypes = [_i32p, _i32p, _u16p, _i32p, _f32p, _f64p] + [ctypes.c_int] * 4
        _lib = L
    return _lib


def ref_available() -> bool:
    return _REF_PATH.exists()


# ---- the reference's own GPU kernels (ref_gpu.cu): configurations by id
REF_GPU_CONFIGS = {
    0: "AqBMMA W2A8 signed   cta<1,48,512> warp<8,24,128> mma<8,8,128> 4 stages (FasterTransformer, M == 1)",
    1: "AqBMMA W2A8 unsigned cta<1,48,512> warp<8,24,128> mma<8,8,128> 4 stages (FasterTransformer, M == 1)",
    2: "AqBMMA W2A8 signed   cta<8,48,256> warp<32,48,128> mma<8,8,128> 5 stages (FasterTransformer, M > 1)",
    3: "AqBMMA W2A8 unsigned cta<8,48,256> warp<32,48,128> mma<8,8,128> 5 stages (FasterTransformer, M > 1)",
    4: "AqBMMA W4A4 signed   cta<2,32,256> warp<8,64,128> mma<8,8,128> 2 stages (engine search space)",
}
_ref_gpu = None


def ref_gpu_available() -> bool:
    return _REF_GPU_PATH.exists()


def ref_gpu() -> ctypes.CDLL:
    global _ref_gpu
    if _ref_gpu is None:
        L = ctypes.CDLL(str(_REF_GPU_PATH))
        L.abq_ref_gpu_gemm.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        L.abq_ref_gpu_gemm.restype = ctypes.c_int
        L.abq_ref_gpu_config.argtypes = [ctypes.c_int] + [ctypes.POINTER(ctypes.c_int)] * 3
        L.abq_ref_gpu_config.restype = ctypes.c_int
        _ref_gpu = L
    return _ref_gpu


_ref_sampled = None


def ref_sampled_available() -> bool:
    return _REF_SAMPLED_PATH.exists()


def ref_sampled() -> ctypes.CDLL:
    """A sample of the reference's own W2A8 / W3A8 / W4A8 decode-tile instantiations (source generated from its lists)."""
    global _ref_sampled
    if _ref_sampled is None:
        L = ctypes.CDLL(str(_REF_SAMPLED_PATH))
        L.abq_ref_sampled_count.restype = ctypes.c_int
        L.abq_ref_sampled_info.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int), ctypes.c_char_p, ctypes.c_int]
        L.abq_ref_sampled_gemm.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                           ctypes.c_int, ctypes.c_void_p]
        _ref_sampled = L
    return _ref_sampled


def ref_sampled_configs():
    """[(index, x_bits, w_bits, name)] of the sampled reference configurations (all signed, one token row per tile)."""
    L = ref_sampled()
    out = []
    for i in range(L.abq_ref_sampled_count()):
        a, b, name = ctypes.c_int(), ctypes.c_int(), ctypes.create_string_buffer(96)
        L.abq_ref_sampled_info(i, ctypes.byref(a), ctypes.byref(b), name, 96)
        out.append((i, a.value, b.value, name.value.decode()))
    return out


def ref_gpu_config(cfg: int):
    """(x_bits, w_bits, signed) of a reference GPU kernel configuration."""
    a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    if not ref_gpu().abq_ref_gpu_config(cfg, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)):
        raise KeyError(cfg)
    return a.value, b.value, bool(c.value)


def ref_gpu_gemm(cfg: int, x_planes_ptr: int, w_planes_ptr: int, M: int, N: int, K: int, out_ptr: int, repeats: int = 1, stream: int = 0):
    """Launch the reference's kernel `cfg` on device pointers (int32 out [M][N]); raises on its own refusal."""
    rc = ref_gpu().abq_ref_gpu_gemm(cfg, x_planes_ptr, w_planes_ptr, M, N, K, out_ptr, repeats, stream)
    if rc != 0:
        raise RuntimeError(f"reference GPU kernel {cfg}: error {rc}")


def ref() -> ctypes.CDLL:
    """The reference's own code (C++ symbols, hence the mangled names)."""
    global _ref
    if _ref is None:
        R = ctypes.CDLL(str(_REF_PATH))
        # void compute_ref(int *w, int *x, int *ref_c, int M, int N, int K, int W_BIT, int X_BIT, bool SIGNED)
        R.compute_ref = getattr(R, "_Z11compute_refPiS_S_iiiiib")
        R.compute_ref.argtypes = [_i32p, _i32p, _i32p] + [ctypes.c_int] * 5 + [ctypes.c_bool]
        R.compute_ref.restype = None
        # void init_matrix(int *matrix, int m, int n, int bits)
        R.init_matrix = getattr(R, "_Z11init_matrixPiiii")
        R.init_matrix.argtypes = [_i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        R.init_matrix.restype = None
        # cudaError_t launch_pack(const int *in, int *out, int m, int k, int BIT, cudaStream_t stream)
        R.launch_pack = getattr(R, "_Z11launch_packPKiPiiiiP11CUstream_st")
        R.launch_pack.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        R.launch_pack.restype = ctypes.c_int
        R.launch_pack4 = getattr(R, "_Z12launch_pack4PKiPiiiiP11CUstream_st")
        R.launch_pack4.argtypes = R.launch_pack.argtypes
        R.launch_pack4.restype = ctypes.c_int
        _ref = R
    return _ref


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def threads() -> int:
    return lib().abq_oracle_threads()


def set_threads(n: int) -> None:
    lib().abq_oracle_set_threads(int(n))


def init_matrix_rand(rows: int, cols: int, bits: int, seed: int | None = None) -> np.ndarray:
    """``rand() % 2^bits`` generator of the reference test driver (seed None keeps the libc state)."""
    if seed is not None:
        lib().abq_oracle_srand(seed)
    out = np.empty((rows, cols), dtype=np.int32)
    lib().abq_oracle_init_matrix(_p(out, _i32p), rows, cols, bits)
    return out


def pack(values: np.ndarray, bits: int) -> np.ndarray:
    """int32 [rows][K] -> uint32 planes [bits][rows][K/32] (element j of a word at bit 31-j)."""
    v = _c(values, np.int32)
    rows, K = v.shape
    assert K % 32 == 0
    out = np.empty((bits, rows, K // 32), dtype=np.uint32)
    lib().abq_oracle_pack(_p(v, _i32p), _p(out, _u32p), rows, K, bits)
    return out


def pack4(nibbles: np.ndarray, rows: int, K: int, bits: int = 4) -> np.ndarray:
    """uint32 words holding 8 nibbles each (first element in the top nibble) -> planes."""
    v = _c(nibbles, np.uint32).reshape(-1)
    assert v.size == rows * K // 8
    out = np.empty((bits, rows, K // 32), dtype=np.uint32)
    lib().abq_oracle_pack4(_p(v, _u32p), _p(out, _u32p), rows, K, bits)
    return out


def unpack(planes: np.ndarray, signed: bool) -> np.ndarray:
    p = _c(planes, np.uint32)
    bits, rows, kw = p.shape
    out = np.empty((rows, kw * 32), dtype=np.int32)
    lib().abq_oracle_unpack(_p(p, _u32p), _p(out, _i32p), rows, kw * 32, bits, int(signed))
    return out


def compute_ref(w_planes: np.ndarray, x_planes: np.ndarray, x_signed: bool, w_signed: bool,
                m0: int = 0, m1: int | None = None) -> np.ndarray:
    """Literal plane/bit loop; returns int32 [M][N] (rows outside [m0, m1) are left zero)."""
    w = _c(w_planes, np.uint32)
    x = _c(x_planes, np.uint32)
    wb, N, kw = w.shape
    xb, M, kw2 = x.shape
    assert kw == kw2
    m1 = M if m1 is None else m1
    out = np.zeros((M, N), dtype=np.int32)
    lib().abq_oracle_compute_ref(_p(w, _u32p), _p(x, _u32p), _p(out, _i32p), M, N, kw * 32, wb, xb,
                                 int(x_signed), int(w_signed), m0, m1)
    return out


def gemm_values(x_vals: np.ndarray, w_vals: np.ndarray) -> np.ndarray:
    """Exact integer GEMM on codes, D = X W^T (int64 accumulate, int32 result)."""
    x = _c(x_vals, np.int32)
    w = _c(w_vals, np.int32)
    M, K = x.shape
    N, K2 = w.shape
    assert K == K2
    out = np.empty((M, N), dtype=np.int32)
    lib().abq_oracle_gemm_values(_p(x, _i32p), _p(w, _i32p), _p(out, _i32p), M, N, K)
    return out


def gemm_values_blas(x_vals: np.ndarray, w_vals: np.ndarray) -> np.ndarray:
    """Same product through float64 BLAS: exact because |sum| <= 255*255*K < 2^53."""
    d = x_vals.astype(np.float64) @ w_vals.astype(np.float64).T
    return d.astype(np.int64).astype(np.int32)


def quantize_half_compat(x_half: np.ndarray, scale: float, bits: int):
    """FasterTransformer wrapper quantiser: int(half(x) * half(scale)), truncating, unclamped."""
    xh = _c(x_half, np.float16)
    rows, K = xh.shape
    planes = np.empty((bits, rows, K // 32), dtype=np.uint32)
    codes = np.empty((rows, K), dtype=np.int32)
    lib().abq_oracle_quantize_half_compat(_p(xh.view(np.uint16), _u16p), float(scale), _p(planes, _u32p),
                                          _p(codes, _i32p), rows, K, bits)
    return planes, codes


def quantize_half_rtn(x_half: np.ndarray, row_scale: np.ndarray, bits: int):
    """Round-to-nearest-even, clamped, per-token scale (quantizer.py semantics)."""
    xh = _c(x_half, np.float16)
    rows, K = xh.shape
    rs = _c(row_scale, np.float32)
    assert rs.size == rows
    planes = np.empty((bits, rows, K // 32), dtype=np.uint32)
    codes = np.empty((rows, K), dtype=np.int32)
    lib().abq_oracle_quantize_half_rtn(_p(xh.view(np.uint16), _u16p), _p(rs, _f32p), _p(planes, _u32p),
                                       _p(codes, _i32p), rows, K, bits)
    return planes, codes


def dequant_tensor_compat(acc: np.ndarray, scale_half: np.float16) -> np.ndarray:
    """FasterTransformer epilogue: half(int acc) * half scale, two fp16 roundings."""
    a = _c(acc, np.int32)
    out = np.empty(a.shape, dtype=np.float16)
    sbits = int(np.array(scale_half, dtype=np.float16).view(np.uint16))
    lib().abq_oracle_dequant_tensor_compat(_p(a, _i32p), sbits, _p(out.view(np.uint16), _u16p), a.size)
    return out


def dequant_gemm(x_vals, w_vals, w_scale_half, w_zero=None, x_scale=None, group: int | None = None) -> np.ndarray:
    """Double-precision scale/zero-point GEMM; w_scale_half is float16 [N][K/group]."""
    x = _c(x_vals, np.int32)
    w = _c(w_vals, np.int32)
    M, K = x.shape
    N = w.shape[0]
    group = K if group is None else group
    ws = _c(w_scale_half, np.float16).reshape(N, K // group)
    wz = None if w_zero is None else _c(w_zero, np.int32).reshape(N, K // group)
    xs = None if x_scale is None else _c(x_scale, np.float32).reshape(M)
    out = np.empty((M, N), dtype=np.float64)
    lib().abq_oracle_dequant_gemm(_p(x, _i32p), _p(w, _i32p), _p(ws.view(np.uint16), _u16p),
                                  None if wz is None else _p(wz, _i32p),
                                  None if xs is None else _p(xs, _f32p),
                                  _p(out, _f64p), M, N, K, group)
    return out


# ---- the reference's own host code (only where oracle/_ref was built) ----

def ref_init_matrix(rows: int, cols: int, bits: int) -> np.ndarray:
    out = np.empty((rows, cols), dtype=np.int32)
    ref().init_matrix(_p(out, _i32p), rows, cols, bits)
    return out


def ref_compute_ref(w_planes: np.ndarray, x_planes: np.ndarray, signed: bool) -> np.ndarray:
    w = _c(w_planes, np.uint32).view(np.int32)
    x = _c(x_planes, np.uint32).view(np.int32)
    wb, N, kw = w.shape
    xb, M, _ = x.shape
    out = np.empty((M, N), dtype=np.int32)
    ref().compute_ref(_p(w, _i32p), _p(x, _i32p), _p(out, _i32p), M, N, kw * 32, wb, xb, bool(signed))
    return out


def quantize_weights_minmax(w_half: np.ndarray, bits: int, group: int | None = None, symmetric: bool = False):
    """Weight quantiser of the reference's PTQ side restated in float32 (algorithm/quantize/quantizer.py:149-179 min/max
    calibration without learnable clipping; :111-132 code rule): returns (codes int32 [N][K], scale fp16 [N][G], zero u8
    [N][G]) with G = K / group (1 for per-channel).  Codes and zero points are clamped into 0 .. 2^bits - 1, the range
    bit-planes can hold (the reference lets 1- and 2-bit codes reach 2^bits, :66-68, and the zero point leave the range)."""
    w = np.ascontiguousarray(w_half, dtype=np.float16).astype(np.float32)
    N, K = w.shape
    g = group if group else K
    x = w.reshape(N, K // g, g)
    lo, hi = x.min(axis=2), x.max(axis=2)
    qmax = np.float32((1 << bits) - 1)
    if symmetric:
        scale = np.maximum(np.abs(lo), np.abs(hi)) / np.float32((1 << (bits - 1)) - 1)
        scale = np.clip(scale, np.float32(1e-5), np.float32(1e4)).astype(np.float32)
        zero = np.full_like(scale, (1 << (bits - 1)) - 1)
    else:
        levels = np.float32((1 << bits) if bits <= 2 else (1 << bits) - 1)
        scale = ((hi - lo).astype(np.float32) / levels).astype(np.float32)
        scale = np.clip(scale, np.float32(1e-5), np.float32(1e4)).astype(np.float32)
        zero = np.rint(np.clip((-lo / scale).astype(np.float32), np.float32(-1e4), np.float32(1e4))).astype(np.float32)
        zero = np.clip(zero, np.float32(0), qmax)
    codes = np.rint((x / scale[:, :, None]).astype(np.float32)).astype(np.float32) + zero[:, :, None]
    codes = np.clip(codes, np.float32(0), qmax).astype(np.int32).reshape(N, K)
    return codes, scale.astype(np.float16), zero.astype(np.uint8)
