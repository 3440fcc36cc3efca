"""torch operators over the C ABI: what the reference's torch extension set out to be.

The reference's extension exports one function, ``mul_w2a8(A, B, C, prob_m, prob_n, prob_k, sms, max_par)``
(algorithm/ABQ/csrc/ABQ_cuda.cu:24-53): it checks ``prob_k >= 128``, builds the op state of one fixed W2A8 instantiation
and returns without ever calling the launch function.  Here:

* ``mul_w2a8``                 -- the same signature and error behaviour, and the GEMM is actually launched
* ``torch.ops.abq_b200.gemm_planes``    -- any WxAy: activation planes x weight planes -> int32 [M][N]
* ``torch.ops.abq_b200.linear_half``    -- fp16 activations (quantised inside the GEMM call with a static scale) x weight
                                           planes -> fp16 [M][N] through the fused per-channel / per-group dequantisation

Both operators are registered with ``torch.library`` (device "cuda" only: there is no CPU kernel, a CPU tensor is an
error) together with shape functions, so they can appear in traced graphs.  Scratch memory comes from torch's caching
allocator, on the current stream.
"""
from __future__ import annotations

import torch

from . import binding as B

_LIB = "abq_b200"


def _workspace(M: int, N: int, K: int, x_bits: int, w_bits: int, device):
    return torch.empty(max(256, B.gemm_workspace_bytes(M, N, K, x_bits, w_bits)), dtype=torch.uint8, device=device)


def _check_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("abq_b200 operators run on CUDA tensors only: there is no CPU path")


@torch.library.custom_op(f"{_LIB}::gemm_planes", mutates_args=(), device_types="cuda")
def gemm_planes(x_planes: torch.Tensor, w_planes: torch.Tensor, x_bits: int, w_bits: int, signed: bool) -> torch.Tensor:
    """x_planes int32 [x_bits][M][K/32], w_planes int32 [w_bits][N][K/32] (the reference's plane format) -> int32 [M][N]."""
    _check_cuda(x_planes, w_planes)
    if x_planes.dim() != 3 or w_planes.dim() != 3 or x_planes.shape[0] != x_bits or w_planes.shape[0] != w_bits or x_planes.shape[2] != w_planes.shape[2]:
        raise RuntimeError(f"plane shapes {tuple(x_planes.shape)} x {tuple(w_planes.shape)} do not fit W{w_bits}A{x_bits}")
    M, N, K = x_planes.shape[1], w_planes.shape[1], x_planes.shape[2] * 32
    out = torch.empty((M, N), dtype=torch.int32, device=x_planes.device)
    work = _workspace(M, N, K, x_bits, w_bits, x_planes.device)
    B.gemm(B.make_params(M, N, K, x_planes.contiguous(), w_planes.contiguous(), out, x_bits=x_bits, w_bits=w_bits, x_signed=signed, w_signed=signed,
                         workspace=work), torch.cuda.current_stream().cuda_stream)
    return out


@gemm_planes.register_fake
def _(x_planes, w_planes, x_bits, w_bits, signed):
    return x_planes.new_empty((x_planes.shape[1], w_planes.shape[1]), dtype=torch.int32)


@torch.library.custom_op(f"{_LIB}::linear_half", mutates_args=(), device_types="cuda")
def linear_half(x: torch.Tensor, w_planes: torch.Tensor, w_scale: torch.Tensor, w_zero: torch.Tensor | None, x_quant_scale: torch.Tensor,
                x_bits: int, w_bits: int, group_size: int) -> torch.Tensor:
    """fp16 x [M][K] -> fp16 [M][N] = ((q(x) . (w - zero)) * w_scale) / x_quant_scale, with q(x) the FasterTransformer
    quantiser of the reference's pack kernel (the fp16 product x * x_quant_scale converted to an integer, kept as a signed
    ``x_bits`` code), unsigned weight codes in ``w_planes`` [w_bits][N][K/32], ``w_scale`` fp16 [N] (group_size 0)
    or [N][K/group_size], ``w_zero`` uint8 of the same shape or None, ``x_quant_scale`` one fp32 on the device."""
    _check_cuda(x, w_planes, w_scale, w_zero, x_quant_scale)
    if x.dtype != torch.float16 or w_scale.dtype != torch.float16:
        raise RuntimeError("linear_half takes fp16 activations and fp16 weight scales")
    M, K = x.shape
    N = w_planes.shape[1]
    if w_planes.shape[0] != w_bits or w_planes.shape[2] * 32 != K:
        raise RuntimeError(f"weight planes {tuple(w_planes.shape)} do not fit W{w_bits} with K = {K}")
    out = torch.empty((M, N), dtype=torch.float16, device=x.device)
    inv = (1.0 / x_quant_scale.to(torch.float32)).expand(M).contiguous()  # per-token factor of the epilogue
    work = _workspace(M, N, K, x_bits, w_bits, x.device)
    B.gemm(B.make_params(M, N, K, x.contiguous(), w_planes.contiguous(), out, x_bits=x_bits, w_bits=w_bits, x_signed=True, w_signed=False,
                         out_dtype=B.OUT_FP16, scale_mode=B.SCALE_GROUP if group_size else B.SCALE_CHANNEL, group_size=group_size,
                         w_scale=w_scale.contiguous(), w_zero=None if w_zero is None else w_zero.contiguous(), x_scale=inv,
                         x_quant_scale=x_quant_scale, flags=B.FLAG_X_HALF, workspace=work), torch.cuda.current_stream().cuda_stream)
    return out


@linear_half.register_fake
def _(x, w_planes, w_scale, w_zero, x_quant_scale, x_bits, w_bits, group_size):
    return x.new_empty((x.shape[0], w_planes.shape[1]), dtype=torch.float16)


def mul_w2a8(A: torch.Tensor, Bm: torch.Tensor, C: torch.Tensor, prob_m: int, prob_n: int, prob_k: int, sms: int = -1, max_par: int = 8) -> None:
    """The reference extension's entry point: A = activation planes (8 bits, signed), Bm = weight planes (2 bits, signed),
    C = int32 [prob_m][prob_n] written in place.  ``sms`` and ``max_par`` are accepted and ignored, as there."""
    del sms, max_par
    if prob_k < 128:
        raise RuntimeError("'abqgemm_cuda' failed: prob_k < 128!")
    _check_cuda(A, Bm, C)
    work = _workspace(prob_m, prob_n, prob_k, 8, 2, A.device)
    try:
        B.gemm(B.make_params(prob_m, prob_n, prob_k, A, Bm, C, x_bits=8, w_bits=2, x_signed=True, w_signed=True, workspace=work),
               torch.cuda.current_stream().cuda_stream)
    except B.AbqError as e:
        raise RuntimeError(f"'abqgemm_cuda' failed due to unsuccessful initialization ({e})") from e
