"""ctypes binding of include/abq_b200.h.  Device buffers are torch CUDA tensors (or raw pointers).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

ROUTE_AUTO, ROUTE_B1_MMA, ROUTE_I8_MMA, ROUTE_I8_UMMA = 0, 1, 2, 3
OUT_INT32, OUT_FP16 = 0, 1
SCALE_NONE, SCALE_TENSOR_COMPAT, SCALE_CHANNEL, SCALE_GROUP = 0, 1, 2, 3
FLAG_PDL = 1
FLAG_WEIGHTS_PREPARED = 2
FLAG_X_HALF = 4

_PKG = Path(__file__).resolve().parent


class AbqError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: abq_status {status} ({_status_string(status)})")


class FusedAllreduce(ctypes.Structure):
    """Mirror of ``abq_fused_allreduce``."""
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("recv", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8),
                ("counter", ctypes.c_void_p), ("rows_cap", ctypes.c_int)]


class GemmParams(ctypes.Structure):
    """Mirror of ``abq_gemm_params`` (field order is part of the ABI)."""
    _fields_ = [
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
        ("X", ctypes.c_void_p), ("W", ctypes.c_void_p), ("C", ctypes.c_void_p), ("D", ctypes.c_void_p),
        ("bias", ctypes.c_int),
        ("x_bits", ctypes.c_int), ("w_bits", ctypes.c_int),
        ("x_signed", ctypes.c_int), ("w_signed", ctypes.c_int),
        ("out_dtype", ctypes.c_int), ("scale_mode", ctypes.c_int), ("group_size", ctypes.c_int),
        ("w_scale", ctypes.c_void_p), ("w_zero", ctypes.c_void_p), ("x_scale", ctypes.c_void_p),
        ("route", ctypes.c_int), ("flags", ctypes.c_int),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("status_word", ctypes.c_void_p),
        ("x_quant_scale", ctypes.c_void_p),
        ("w_prepared", ctypes.c_void_p),
        ("allreduce", ctypes.POINTER(FusedAllreduce)),
        ("residual", ctypes.c_void_p),
    ]


class GemmState(ctypes.Structure):
    """Mirror of ``abq_gemm_state``."""
    _fields_ = [
        ("p", GemmParams),
        ("init_success", ctypes.c_int), ("route", ctypes.c_int),
        ("grid", ctypes.c_int * 3), ("block", ctypes.c_int * 3), ("cluster", ctypes.c_int),
        ("shared_mem_size", ctypes.c_size_t),
        ("tile", ctypes.c_int * 4),
        ("tmap", (ctypes.c_ulonglong * 16) * 3),
        ("ar", FusedAllreduce),
    ]


_lib = None


def lib_path() -> Path:
    return _PKG / "lib" / "libabq_b200.so"


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = lib_path()
        if not path.exists():
            raise FileNotFoundError(f"{path} is missing: run `python abq-llm_b200/build.py` (no fallback exists)")
        L = ctypes.CDLL(str(path))
        L.abq_version.restype = ctypes.c_char_p
        L.abq_status_string.restype = ctypes.c_char_p
        L.abq_status_string.argtypes = [ctypes.c_int]
        L.abq_last_cuda_error.restype = ctypes.c_int
        L.abq_gemm_workspace_bytes.restype = ctypes.c_size_t
        L.abq_gemm_workspace_bytes.argtypes = [ctypes.c_int] * 6
        L.abq_gemm_prepared_weight_bytes.restype = ctypes.c_size_t
        L.abq_gemm_prepared_weight_bytes.argtypes = [ctypes.POINTER(GemmParams)]
        L.abq_gemm_init.argtypes = [ctypes.POINTER(GemmParams), ctypes.POINTER(GemmState)]
        L.abq_gemm_exec.argtypes = [ctypes.POINTER(GemmState), ctypes.c_void_p]
        L.abq_gemm_prepare_weights.argtypes = [ctypes.POINTER(GemmState), ctypes.c_void_p]
        L.abq_gemm.argtypes = [ctypes.POINTER(GemmParams), ctypes.c_void_p]
        L.abq_gemm_static_scratch.argtypes = [ctypes.POINTER(GemmParams), ctypes.c_void_p]
        L.abq_pack_int32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        L.abq_pack_int4.argtypes = L.abq_pack_int32.argtypes
        L.abq_quantize_pack_half.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                             ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        L.abq_quantize_weights_half.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        L.abq_swiglu_half.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        L.abq_add_half.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p]
        L.abq_rmsnorm_quantize_pack_half.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_float] + [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4 + [ctypes.c_void_p]
        L.abq_unpack_int8.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_void_p]
        _lib = L
    return _lib


def _status_string(s: int) -> str:
    try:
        return lib().abq_status_string(s).decode()
    except Exception:  # library missing: still give a message
        return "?"


def version() -> str:
    return lib().abq_version().decode()


def _ptr(t) -> int | None:
    """Device address of a torch tensor, an int, or None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    assert t.is_cuda and t.is_contiguous(), "device buffers must be contiguous CUDA tensors"
    return t.data_ptr()


def _stream(stream) -> int | None:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _check(status: int, what: str) -> None:
    if status != 0:
        extra = ""
        if status == 4:
            extra = f" [cudaError {lib().abq_last_cuda_error()}]"
        raise AbqError(status, what + extra)


def gemm_workspace_bytes(M: int, N: int, K: int, x_bits: int, w_bits: int, route: int = ROUTE_AUTO) -> int:
    return int(lib().abq_gemm_workspace_bytes(M, N, K, x_bits, w_bits, route))


def make_params(M, N, K, X, W, D, *, x_bits, w_bits, x_signed, w_signed, out_dtype=OUT_INT32, scale_mode=SCALE_NONE,
                group_size=0, C=None, w_scale=None, w_zero=None, x_scale=None, route=ROUTE_AUTO, flags=0, workspace=None,
                status_word=None, x_quant_scale=None, w_prepared=None, allreduce=None, residual=None) -> GemmParams:
    p = GemmParams()
    p.M, p.N, p.K = M, N, K
    p.X, p.W, p.C, p.D = _ptr(X), _ptr(W), _ptr(C), _ptr(D)
    p.bias = 0
    p.x_bits, p.w_bits, p.x_signed, p.w_signed = x_bits, w_bits, int(x_signed), int(w_signed)
    p.out_dtype, p.scale_mode, p.group_size = out_dtype, scale_mode, group_size
    p.w_scale, p.w_zero, p.x_scale = _ptr(w_scale), _ptr(w_zero), _ptr(x_scale)
    p.route, p.flags = route, flags
    p.workspace = _ptr(workspace)
    p.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    p.status_word = _ptr(status_word)
    p.x_quant_scale = _ptr(x_quant_scale)
    p.w_prepared = _ptr(w_prepared)
    p.residual = _ptr(residual)
    # the block carries raw pointers: keep the tensors alive as long as it lives (a temporary passed inline would otherwise
    # be freed, and its memory reused, before the launch)
    p._keep_alive = (X, W, D, C, w_scale, w_zero, x_scale, workspace, status_word, x_quant_scale, w_prepared, residual)
    if allreduce is not None:
        p.allreduce = ctypes.pointer(allreduce)
        p._keep_allreduce = allreduce  # the struct must outlive the call that reads it
    return p


def make_fused_allreduce(world: int, rank: int, recv_ptrs, flag_ptrs, counter, rows_cap: int) -> FusedAllreduce:
    """``recv_ptrs`` / ``flag_ptrs``: every rank's receive buffer / flag array as mapped into this process (ints)."""
    d = FusedAllreduce()
    d.world, d.rank, d.rows_cap = world, rank, rows_cap
    for r in range(world):
        d.recv[r] = int(recv_ptrs[r])
        d.flags[r] = int(flag_ptrs[r])
    d.counter = _ptr(counter)
    return d


def gemm_prepared_weight_bytes(params: GemmParams) -> int:
    """Bytes of the re-ordered weight copy a decode-shape plan reads through ``w_prepared`` (0: no prepared form)."""
    return int(lib().abq_gemm_prepared_weight_bytes(ctypes.byref(params)))


def state_kernel(state: GemmState) -> str:
    """Name of the GEMM kernel a plan launches (for reports): the route, and on the decode route which of its two kernels."""
    if state.route == ROUTE_I8_MMA:
        return "stream_kernel" if (state.tmap[1][0] & 0xffffffff) == 0x5354524d else "decode_kernel"
    return {ROUTE_B1_MMA: "b1_kernel", ROUTE_I8_UMMA: "umma_kernel"}.get(state.route, "?")


def gemm_init(params: GemmParams) -> GemmState:
    st = GemmState()
    _check(lib().abq_gemm_init(ctypes.byref(params), ctypes.byref(st)), "abq_gemm_init")
    return st


def gemm_exec(state: GemmState, stream=None) -> None:
    _check(lib().abq_gemm_exec(ctypes.byref(state), _stream(stream)), "abq_gemm_exec")


def gemm_prepare_weights(state: GemmState, stream=None) -> None:
    _check(lib().abq_gemm_prepare_weights(ctypes.byref(state), _stream(stream)), "abq_gemm_prepare_weights")


def peer_allreduce_half(bufs_dev: int, signals_dev: int, rank: int, world: int, signal_offset: int, out, n_halves: int, counter,
                        status_word=None, stream=None, residual=None) -> None:
    """One-shot sum over the ranks' partial buffers (peer-mapped pointers, see abq_peer_allreduce_half), plus ``residual``."""
    f = lib().abq_peer_allreduce_half
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p,
                  ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    _check(f(bufs_dev, signals_dev, rank, world, signal_offset, _ptr(out), n_halves, _ptr(counter), _ptr(status_word), _ptr(residual),
             _stream(stream)), "abq_peer_allreduce_half")


def gemm(params: GemmParams, stream=None) -> None:
    _check(lib().abq_gemm(ctypes.byref(params), _stream(stream)), "abq_gemm")


STATIC_SCRATCH_BYTES = 16 << 20


def gemm_static_scratch(params: GemmParams, stream=None) -> None:
    """abq_gemm on the library's built-in device scratch array: allocates nothing, ignores params.workspace."""
    _check(lib().abq_gemm_static_scratch(ctypes.byref(params), _stream(stream)), "abq_gemm_static_scratch")


def pack_int32(values, planes, rows: int, K: int, bits: int, stream=None) -> None:
    _check(lib().abq_pack_int32(_ptr(values), _ptr(planes), rows, K, bits, _stream(stream)), "abq_pack_int32")


def pack_int4(nibbles, planes, rows: int, K: int, bits: int = 4, stream=None) -> None:
    _check(lib().abq_pack_int4(_ptr(nibbles), _ptr(planes), rows, K, bits, _stream(stream)), "abq_pack_int4")


def quantize_pack_half(x_half, scale, planes, rows: int, K: int, bits: int, mode: int = 0, stream=None) -> None:
    _check(lib().abq_quantize_pack_half(_ptr(x_half), _ptr(scale), _ptr(planes), rows, K, bits, mode, _stream(stream)),
           "abq_quantize_pack_half")


def rmsnorm_quantize_pack_half(x_half, gamma, eps: float, rows: int, K: int, bits: int, mode: int, *, residual=None, sum_out=None, scale=None,
                               row_scale_out=None, planes=None, y_out=None, stream=None) -> None:
    """(residual add ->) RMSNorm -> quantiser -> planes in one launch; see abq_rmsnorm_quantize_pack_half in the header."""
    _check(lib().abq_rmsnorm_quantize_pack_half(_ptr(x_half), _ptr(residual), _ptr(sum_out), _ptr(gamma), ctypes.c_float(eps), _ptr(scale),
                                                _ptr(row_scale_out), _ptr(planes), _ptr(y_out), rows, K, bits, mode, _stream(stream)),
           "abq_rmsnorm_quantize_pack_half")


def quantize_weights_half(w_half, planes, scale, zero, N: int, K: int, bits: int, group_size: int = 0, symmetric: bool = False, stream=None) -> None:
    """fp16 weights [N][K] -> bit-planes + fp16 scale + u8 zero point (min/max calibration of the reference's quantiser)."""
    _check(lib().abq_quantize_weights_half(_ptr(w_half), N, K, bits, group_size, int(symmetric), _ptr(planes), _ptr(scale), _ptr(zero), _stream(stream)),
           "abq_quantize_weights_half")


def swiglu_half(gate_up, out, M: int, F: int, stream=None) -> None:
    """out[m][f] = silu(gate_up[m][f]) * gate_up[m][F + f]: one launch, in the GEMMs' dependent-launch chain."""
    _check(lib().abq_swiglu_half(_ptr(gate_up), _ptr(out), M, F, _stream(stream)), "abq_swiglu_half")


def add_half(a, b, out, n: int, stream=None) -> None:
    _check(lib().abq_add_half(_ptr(a), _ptr(b), _ptr(out), n, _stream(stream)), "abq_add_half")


def unpack_int8(planes, out_i8, rows: int, K: int, bits: int, signed: bool, stream=None) -> None:
    _check(lib().abq_unpack_int8(_ptr(planes), _ptr(out_i8), rows, K, bits, int(signed), _stream(stream)), "abq_unpack_int8")
