"""The C-ABI library without a GPU: it loads, exports every symbol include/abq_b200.h declares, sizes agree with the
Python mirror, and argument validation answers before anything touches a device."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "abq_b200.h").read_text()
    return sorted(set(re.findall(r"ABQ_API\s+[\w\s\*]+?\b(abq_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(abq):
    names = declared_symbols()
    assert len(names) >= 12 and "abq_gemm_init" in names and "abq_gemm_static_scratch" in names
    lib = abq.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in abq_b200.h but not exported"


def test_struct_sizes_match_the_header(abq, tmp_path):
    src = tmp_path / "sz.c"
    src.write_text('#include "abq_b200.h"\n#include <stdio.h>\nint main(void){printf("%zu %zu\\n", sizeof(abq_gemm_params), sizeof(abq_gemm_state));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)  # the header is plain C
    a, b = (int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split())
    assert a == ctypes.sizeof(abq.GemmParams) and b == ctypes.sizeof(abq.GemmState)


def test_version_and_status_strings(abq):
    assert "sm_100a" in abq.version()
    assert abq.lib().abq_status_string(3).decode().startswith("workspace")


def test_validation_needs_no_device(abq):
    from abq_llm_b200 import binding as B
    p = B.GemmParams()
    st = B.GemmState()
    init = abq.lib().abq_gemm_init
    assert init(None, ctypes.byref(st)) == 1
    p.M, p.N, p.K = 1, 64, 128
    assert init(ctypes.byref(p), ctypes.byref(st)) == 1  # null operand pointers
    p.X = p.W = p.D = 4096
    p.x_bits, p.w_bits = 8, 2
    p.K = 100
    assert init(ctypes.byref(p), ctypes.byref(st)) == 1  # K % 128 != 0 (engine/test_any_mma.cu:99)
    p.K = 128
    p.bias = 1
    assert init(ctypes.byref(p), ctypes.byref(st)) == 2  # bias is unsupported, as in the reference (aq_bmma_op.h:79)
    p.bias = 0
    p.w_bits = 9
    assert init(ctypes.byref(p), ctypes.byref(st)) == 1
    p.w_bits = 2
    p.out_dtype, p.scale_mode = 1, 3  # fp16 + group scales without a scale pointer
    assert init(ctypes.byref(p), ctypes.byref(st)) == 1
    p.out_dtype, p.scale_mode = 0, 0
    p.flags = abq.FLAG_X_HALF            # fp16 activations: need the quantiser scale and signed codes
    assert init(ctypes.byref(p), ctypes.byref(st)) == 1
    p.x_quant_scale, p.x_signed, p.route = 4096, 1, abq.ROUTE_B1_MMA
    assert init(ctypes.byref(p), ctypes.byref(st)) == 2  # the 1-bit route multiplies planes
    p.flags, p.route = 0, 0
    p.M = 0
    assert init(ctypes.byref(p), ctypes.byref(st)) == 1  # empty problem
    assert st.init_success == 0
    assert abq.lib().abq_gemm_exec(ctypes.byref(st), None) == 5  # not initialised
    assert abq.lib().abq_gemm_prepare_weights(ctypes.byref(st), None) == 5
    assert abq.lib().abq_pack_int32(None, None, 1, 128, 4, None) == 1


def test_misaligned_pointers_are_argument_errors(abq):
    """Operands and results move in 16-byte pieces; a pointer that is not 16-byte aligned (a tensor view at an element
    offset) must come back as a status, not as a fault on the device.  Nothing is launched here."""
    from abq_llm_b200 import binding as B
    L = abq.lib()
    p, st = B.GemmParams(), B.GemmState()
    p.M, p.N, p.K, p.x_bits, p.w_bits = 1, 64, 128, 8, 2
    for bad in ("X", "W", "D"):
        p.X = p.W = p.D = 4096
        setattr(p, bad, 4096 + 4)
        assert L.abq_gemm_init(ctypes.byref(p), ctypes.byref(st)) == 1, bad
    assert L.abq_pack_int32(4096 + 4, 8192, 1, 128, 4, None) == 1
    assert L.abq_pack_int32(4096, 8192 + 8, 1, 128, 4, None) == 1
    assert L.abq_pack_int4(4096 + 2, 8192, 1, 128, 4, None) == 1
    assert L.abq_quantize_pack_half(4096 + 2, 4096, 8192, 1, 128, 8, 0, None) == 1
    assert L.abq_unpack_int8(4096, 8192 + 1, 1, 128, 8, 1, None) == 1


def test_static_scratch_refuses_prepared_weights_without_a_device(abq):
    from abq_llm_b200 import binding as B
    p = B.GemmParams()
    p.M, p.N, p.K, p.x_bits, p.w_bits = 64, 64, 128, 4, 4
    p.X = p.W = p.D = 4096
    p.flags = abq.FLAG_WEIGHTS_PREPARED
    assert abq.lib().abq_gemm_static_scratch(ctypes.byref(p), None) == 1


def test_workspace_sizes(abq):
    assert abq.gemm_workspace_bytes(1, 4096, 4096, 8, 2) % 256 == 0
    big = abq.gemm_workspace_bytes(4096, 4096, 4096, 8, 8)
    assert big >= 2 * 4096 * 4096  # expanded int8 copies of both operands
    assert big > abq.STATIC_SCRATCH_BYTES


def test_missing_library_fails_loudly(abq, monkeypatch, tmp_path):
    from abq_llm_b200 import binding as B
    monkeypatch.setattr(B, "_lib", None)
    monkeypatch.setattr(B, "lib_path", lambda: tmp_path / "nope.so")
    with pytest.raises(FileNotFoundError):
        B.lib()


def test_torch_operators_are_registered_and_refuse_cpu_tensors(abq):
    """abq_b200::gemm_planes / linear_half exist after importing the operator module, have shape functions (a traced graph
    can hold them) and have no CPU kernel: a CPU tensor is an error, not a silent fallback."""
    import importlib
    import torch
    importlib.import_module("abq_llm_b200.torch_ops")
    assert hasattr(torch.ops.abq_b200, "gemm_planes") and hasattr(torch.ops.abq_b200, "linear_half")
    x = torch.zeros((8, 1, 4), dtype=torch.int32)
    w = torch.zeros((2, 16, 4), dtype=torch.int32)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.abq_b200.gemm_planes(x, w, 8, 2, True)
    meta = torch.ops.abq_b200.gemm_planes(x.to("meta"), w.to("meta"), 8, 2, True)
    assert tuple(meta.shape) == (1, 16) and meta.dtype == torch.int32
