"""Python mirror of the reference's host-side interface for this path.

* ``launch_pack`` / ``launch_pack4``  -- engine/common/pack.h:20-24
* ``ABQGEMMWrapper``                  -- fastertransformer/src/fastertransformer/kernels/abqgemm/abq_gemm_wrapper.h:6-32

Same names and argument meaning; device buffers are torch CUDA tensors.  Errors raise instead of the
reference's printf-and-return (abq_gemm_wrapper.cu:100-103,128-136).
"""
from __future__ import annotations

from . import binding as B


def launch_pack(in_data, pack_data, m: int, k: int, BIT: int, stream=None) -> None:
    """int32-per-value [m][k] -> planes[BIT][m][k/32]."""
    B.pack_int32(in_data, pack_data, m, k, BIT, stream)


def launch_pack4(in_data, pack_data, m: int, k: int, BIT: int, stream=None) -> None:
    """nibble-packed int4 (m*k/8 int32 words) -> planes[BIT][m][k/32]."""
    B.pack_int4(in_data, pack_data, m, k, BIT, stream)


class ABQGEMMWrapper:
    """``ABQGEMMWrapper(X_BITS, W_BITS, SIGNED)`` with ``pack`` and ``gemm`` as in the reference.

    ``gemm`` quantises + packs the fp16 activations into the caller's workspace (compat quantiser:
    ``int(half(x) * half(scale))``), then multiplies by the pre-packed weight planes ``B`` and writes
    ``D = half(acc) * half(scale_out)``.  ``scale_out`` is a device float whose first two bytes are read
    as fp16, as the reference does (abq_gemm_wrapper.cu:125-126: ``reinterpret_cast<const half*>(scale_out)``).
    Unlike the reference, any W/A bit width from 1 to 8 is accepted, and the workspace size is checked.
    """

    def __init__(self, X_BITS: int, W_BITS: int, SIGNED: bool):
        self.x_bits_, self.w_bits_, self.signed_ = X_BITS, W_BITS, bool(SIGNED)

    def workspace_bytes(self, M: int, N: int, K: int) -> int:
        planes = self.x_bits_ * M * (K // 32) * 4
        planes = (planes + 255) & ~255
        return planes + B.gemm_workspace_bytes(M, N, K, self.x_bits_, self.w_bits_)

    def pack(self, in_data, packed_data, M: int, K: int, BIT: int, stream=None, scale=None) -> None:
        if scale is None:
            B.pack_int32(in_data, packed_data, M, K, BIT, stream)
        else:
            B.quantize_pack_half(in_data, scale, packed_data, M, K, BIT, 0, stream)

    def gemm(self, M, N, K, A, B_planes, C, D, scale, scale_inter, scale_out, bias, abq_gemm_workspace, abq_gemm_ws_bytes,
             stream=None) -> None:
        if K < 128 or K % 128 != 0:
            raise B.AbqError(1, f"[ABQ][Error] unsupport K = {K}")
        need = self.workspace_bytes(M, N, K)
        if abq_gemm_ws_bytes < need:
            raise B.AbqError(3, f"workspace of {abq_gemm_ws_bytes} bytes, {need} needed")
        ws = abq_gemm_workspace
        base = ws.data_ptr()
        # signed configurations: the GEMM call quantises the fp16 activations itself (same codes as pack, one launch less)
        fused = self.signed_
        plane_bytes = 0 if fused else (self.x_bits_ * M * (K // 32) * 4 + 255) & ~255
        if not fused:
            B.quantize_pack_half(A, scale, base, M, K, self.x_bits_, 0, stream)
        p = B.GemmParams()
        p.M, p.N, p.K = M, N, K
        p.X, p.W, p.C, p.D = (B._ptr(A) if fused else base), B._ptr(B_planes), B._ptr(scale_out), B._ptr(D)
        p.flags = B.FLAG_X_HALF if fused else 0
        p.x_quant_scale = B._ptr(scale)
        p.bias = int(bool(bias))
        p.x_bits, p.w_bits = self.x_bits_, self.w_bits_
        p.x_signed = p.w_signed = int(self.signed_)
        p.out_dtype, p.scale_mode = B.OUT_FP16, B.SCALE_TENSOR_COMPAT
        p.workspace = base + plane_bytes
        p.workspace_bytes = abq_gemm_ws_bytes - plane_bytes
        B.gemm(p, stream)
