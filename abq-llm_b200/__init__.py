"""B200 (sm_100a) arbitrary-bit quantized GEMM engine: Python host side over the C ABI.

The directory name contains a hyphen, so import it through ``importlib`` (tests/conftest.py and
__graft_entry__.py register it as ``abq_llm_b200``).
"""
from .binding import (  # noqa: F401
    ROUTE_AUTO, ROUTE_B1_MMA, ROUTE_I8_MMA, ROUTE_I8_UMMA,
    OUT_INT32, OUT_FP16, SCALE_NONE, SCALE_TENSOR_COMPAT, SCALE_CHANNEL, SCALE_GROUP, FLAG_PDL, FLAG_WEIGHTS_PREPARED, FLAG_X_HALF,
    AbqError, GemmParams, GemmState, FusedAllreduce, make_fused_allreduce, lib, lib_path, version,
    gemm_workspace_bytes, gemm_prepared_weight_bytes, state_kernel, gemm_init, gemm_exec, gemm_prepare_weights, gemm, gemm_static_scratch, STATIC_SCRATCH_BYTES,
    pack_int32, pack_int4, quantize_pack_half, quantize_weights_half, swiglu_half, add_half, rmsnorm_quantize_pack_half, unpack_int8, peer_allreduce_half,
)
from .wrapper import ABQGEMMWrapper, launch_pack, launch_pack4  # noqa: F401
