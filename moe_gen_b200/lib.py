"""ctypes binding of libmoegen_b200.so (the C ABI declared in include/moegen_b200.h).

There is no fallback: if the shared library is missing or a call fails, a
RuntimeError is raised, as C++ exceptions from the reference's pybind module
surface in Python (core/utils.h:71-83 CUDA_CHECK -> std::runtime_error).
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# MOEGEN_B200_LIB selects another build of the same library (the -DMG_BOUNDS_CHECK one, for test runs)
LIB_PATH = os.environ.get("MOEGEN_B200_LIB") or os.path.join(_PKG, "libmoegen_b200.so")

GATE_SOFTMAX_GREEDY, GATE_SOFTMAX_GROUP_MAX, GATE_SIGMOID_NOAUX_TC, GATE_SOFTMAX_TOPK_RENORM = 0, 1, 2, 3
COMBINE_FP32, COMBINE_BF16_PROD, COMBINE_BF16_SEQ = 0, 1, 2
WEIGHT_BF16, WEIGHT_FP8_BLOCK128 = 0, 1
DEV_OK, DEV_WAIT_TIMEOUT, DEV_CAPACITY, DEV_BOUNDS = 0, 1, 2, 3
OPT_FP8_MODE = 1
OPT_PAIR_GEMM = 2
OPT_KEEP_DEQUANT = 3
OPT_FP8_M256 = 4
OPT_BATCH_TOKENS = 5
OPT_SHARED_EARLY = 6
OPT_RING_BYTES = 7
OPT_RING_PERSIST = 8
OPT_ROWS_BOUND = 9
OPT_ROUTE_FIXUP = 10
FP8_AUTO, FP8_PREDEQUANT, FP8_IN_KERNEL, FP8_RING = 0, 1, 2, 3


class LayerDesc(C.Structure):
    _fields_ = [("struct_bytes", C.c_int32), ("hidden", C.c_int32), ("inter", C.c_int32),
                ("inter_shared", C.c_int32), ("n_experts", C.c_int32), ("top_k", C.c_int32),
                ("n_group", C.c_int32), ("topk_group", C.c_int32), ("gating", C.c_int32),
                ("norm_topk_prob", C.c_int32), ("routed_scale", C.c_float),
                ("weight_format", C.c_int32), ("combine_mode", C.c_int32),
                ("ep_rank", C.c_int32), ("ep_size", C.c_int32)]


_vp, _i64, _i32, _sz = C.c_void_p, C.c_int64, C.c_int32, C.c_size_t
_P = C.POINTER

# name -> argtypes; every function returns int except mg_last_error
SIGNATURES = {
    "mg_create": [_P(LayerDesc), _P(_vp)],
    "mg_destroy": [_vp],
    "mg_device_status": [_vp, _P(_i32), _P(_i32)],
    "mg_device_status_async": [_vp, _vp, _vp],
    "mg_l2_set_aside": [_sz, _P(_sz)],
    "mg_packed_weight_bytes": [_vp, _P(_sz)],
    "mg_workspace_bytes": [_vp, _i64, _i64, _P(_sz)],
    "mg_padded_rows": [_vp, _i64, _P(_i64)],
    "mg_pack_expert": [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "mg_dequant_fp8_block128": [_vp, _vp, _i64, _i64, _vp, _vp],
    "mg_gate_logits": [_vp, _vp, _vp, _i64, _vp, _vp],
    "mg_route_topk": [_vp, _vp, _vp, _i64, _vp, _vp, _vp],
    "mg_gate_route_topk": [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp],
    "mg_route_fix_bytes": [_i64, _P(_sz)],
    "mg_plan_ws_bytes": [_vp, _i64, _P(_sz)],
    "mg_permute_plan": [_vp, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp],
    "mg_permute_plan_static": [_vp, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp],
    "mg_permute_rows": [_vp, _vp, _vp, _i64, _vp, _vp],
    "mg_dequant_ws_bytes": [_vp, _P(_sz)],
    "mg_dequant_start": [_vp, _vp, _vp, _vp],
    "mg_expert_ffn": [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp],
    "mg_shared_ffn": [_vp, _vp, _i64, _vp, _vp, _vp, _vp],
    "mg_combine": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp],
    "mg_moe_forward": [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _sz, _vp, _vp],
    "mg_host_chunk_plan": [_i64, _i64, _P(_i64), _i32, _P(_i32)],
    "mg_host_workspace_bytes": [_vp, _i64, _i64, _P(_sz)],
    "mg_moe_forward_host": [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _sz, _vp, _i64, _vp],
    "mg_moe_forward_from_logits": [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _sz, _vp, _vp],
    "mg_workspace_ptr": [_vp, _vp, _i64, _i64, _i32, _P(_vp)],
    "mg_selftest_wait_timeout": [_vp, _i32, _vp],
    "mg_last_launch_count": [_vp, _P(_i32)],
    "mg_ep_alloc": [_sz, _P(_vp)],
    "mg_ep_free": [_vp],
    "mg_ep_export": [_vp, _vp],
    "mg_ep_import": [_vp, _P(_vp)],
    "mg_ep_unimport": [_vp],
    "mg_ep_count": [_vp, _vp, _i64, _vp, _vp, _vp],
    "mg_ep_place": [_vp, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp],
    "mg_ep_dispatch": [_vp, _vp, _vp, _i64, _P(_vp), _vp],
    "mg_ep_dispatch_dedup": [_vp, _vp, _vp, _i64, _P(_vp), _P(_vp), _vp],
    "mg_ep_dispatch_back": [_vp, _vp, _vp, _i64, _P(_vp), _P(_vp), _P(_vp), _vp],
    "mg_ep_expert_ffn_return": [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _P(_vp), _i32, _vp],
    "mg_ep_combine_slots": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp],
    "mg_ep_expert_ffn_copy_return": [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp],
    "mg_ep_mirror_delta": [_vp, _vp, _vp, _vp],
    "mg_ep_combine_mirror": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp],
    "mg_ep_clear_duplicates": [_vp, _vp, _i64, _vp],
    "mg_ep_fill_duplicates": [_vp, _vp, _vp, _i64, _vp],
    "mg_ep_combine": [_vp, _P(_vp), _vp, _vp, _vp, _vp, _i64, _vp, _vp],
    "mg_rmsnorm": [_vp, _vp, _vp, C.c_float, _i64, _vp, _vp],
    "mg_moe_block_forward": [_vp, _vp, _vp, C.c_float, _i64, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp],
    "mg_set_option": [_vp, _i32, _i32],
    "mg_set_stage_timing": [_vp, _i32],
    "mg_stage_times": [_vp, _P(C.c_float), _i32],
}

STAGES = ["gate_logits", "route_topk", "permute_plan", "permute_rows", "dequant", "expert_gemm1",
          "expert_gemm2", "shared_gemm1", "shared_gemm2", "combine"]

_lib = None


def load() -> C.CDLL:
    """Loads the shared library (building nothing).  Raises if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m moe_gen_b200.build` "
                "(there is no CPU or PyTorch fallback for this library)")
        lib = C.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = C.c_int
        lib.mg_last_error.argtypes = []
        lib.mg_last_error.restype = C.c_char_p
        _lib = lib
    return _lib


class MoeGenError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"moegen_b200 error {code}: {text}")
        self.code = code


def check(rc: int) -> None:
    if rc != 0:
        raise MoeGenError(rc, load().mg_last_error().decode("utf-8", "replace"))
