"""Shared helpers of the GPU parity tests: seeded inputs and calls through the C ABI."""
from __future__ import annotations

import numpy as np
import torch


def rand_codes(rng, rows, K, bits, signed):
    if signed:
        return rng.integers(-(1 << (bits - 1)), 1 << (bits - 1), size=(rows, K), dtype=np.int32)
    return rng.integers(0, 1 << bits, size=(rows, K), dtype=np.int32)


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def planes_dev(oracle, codes, bits):
    """Bit-planes of integer codes (two's complement low bits), on the device as int32 words."""
    return dev(oracle.pack(codes, bits).view(np.int32))


def run_gemm(abq, xp, wp, M, N, K, *, x_bits, w_bits, x_signed, w_signed, route=0, out_fp16=False, scale_mode=0, group_size=0,
             C=None, w_scale=None, w_zero=None, x_scale=None, flags=0, env=None):
    """One GEMM through abq_gemm_init / abq_gemm_exec; returns (numpy result, state)."""
    out = torch.full((M, N), -7, dtype=torch.float16 if out_fp16 else torch.int32, device="cuda")
    ws_bytes = max(256, abq.gemm_workspace_bytes(M, N, K, x_bits, w_bits, route))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    from abq_llm_b200 import binding as B
    p = B.make_params(M, N, K, xp, wp, out, x_bits=x_bits, w_bits=w_bits, x_signed=x_signed, w_signed=w_signed,
                      out_dtype=abq.OUT_FP16 if out_fp16 else abq.OUT_INT32, scale_mode=scale_mode, group_size=group_size, C=C,
                      w_scale=w_scale, w_zero=w_zero, x_scale=x_scale, route=route, flags=flags, workspace=ws, status_word=status)
    st = abq.gemm_init(p)
    abq.gemm_exec(st)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device status word {int(status.item())}"
    return out.cpu().numpy(), st
