"""Loads libstrixite_b200.so and declares the C ABI of include/strixite_b200.h for ctypes.

There is no fallback: if the library is missing or a symbol is absent, importing this module raises. Every call
goes through `call()`, which turns a nonzero return code into StrixError carrying strix_last_error().
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libstrixite_b200.so")


class StrixError(RuntimeError):
    """An argument check or a CUDA call failed inside the library (strixite's strix::Error across the C ABI)."""


class QView(C.Structure):
    """strix_qview: field for field strixite runtime/q4_device.hpp:13-18."""

    _fields_ = [("q", C.c_void_p), ("scale", C.c_void_p), ("minv", C.c_void_p), ("N", C.c_int64), ("K", C.c_int64), ("G", C.c_int64)]


class QMixView(C.Structure):
    """strix_qmix_view: an expert stack with a format per expert."""

    _fields_ = [("q", C.c_void_p), ("scale", C.c_void_p), ("minv", C.c_void_p), ("bits", C.c_void_p), ("q_off", C.c_void_p),
                ("E", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("G", C.c_int64)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "strixite_b200: %s is missing - build it with `python strixite_b200/build.py` (needs nvcc). "
            "There is no CPU fallback." % LIB_PATH
        )
    return C.CDLL(LIB_PATH)


lib = _load()

_vp, _i64, _i32, _u32, _int, _sz = C.c_void_p, C.c_int64, C.c_int32, C.c_uint32, C.c_int, C.c_size_t
_qv, _qm = C.POINTER(QView), C.POINTER(QMixView)

# name -> argument types; every function returns int unless listed in _RESTYPES.
SIGNATURES = {
    "strix_quantize": [_int, _vp, _i64, _i64, _i64, _vp, _vp, _vp],
    "strix_dequantize": [_int, _vp, _vp, _vp, _i64, _i64, _i64, _vp],
    "strix_check_qweight": [_int, _i64, _i64, _i64, _sz, _sz, _sz],
    "strix_row_bytes": [_int, _i64],
    "strix_quantize_device": [_int, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp],
    "strix_moe_router": [_vp, _i64, _i64, _i64, _i64, _vp, _i64, _i32, _vp, _vp, _int, _vp, _vp],
    "strix_check_router_error": [_vp, C.c_char_p],
    "strix_report_router_error": [_vp, C.c_char_p],
    "strix_moe_shared_add": [_vp, _vp, _vp, _i64, _i64, _i64, _u32, _int, _vp, _vp],
    "strix_moe_shared_add_inject": [_vp, _vp, _vp, _i64, _i64, _i64, _u32, _vp, _vp, _i64, _int, _vp, _vp],
    "strix_linear_q4": [_vp, _qv, _vp, _i64, _int, _int, _vp],
    "strix_linear_q5": [_vp, _qv, _vp, _i64, _int, _int, _vp],
    "strix_linear_q6": [_vp, _qv, _vp, _i64, _int, _int, _vp],
    "strix_linear_q8": [_vp, _qv, _vp, _i64, _int, _int, _vp],
    "strix_linear_bf16w": [_vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp],
    "strix_linear_q4_wmma": [_vp, _qv, _vp, _i64, _int, _int, _vp],
    "strix_linear_q5_wmma": [_vp, _qv, _vp, _i64, _int, _int, _vp],
    "strix_linear_q6_wmma": [_vp, _qv, _vp, _i64, _int, _int, _vp],
    "strix_linear_q8_wmma": [_vp, _qv, _vp, _i64, _int, _int, _vp],
    "strix_linear_bf16w_wmma": [_vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp],
    "strix_linear_f32w": [_vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp],
    "strix_swiglu": [_vp, _vp, _i64, _i64, _int, _vp],
    "strix_residual_add": [_vp, _vp, _i64, _int, _vp],
    "strix_hc_inject": [_vp, _vp, _vp, _i64, _i64, _i64, _int, _vp],
    "strix_hc_mix_down": [_vp, _qv, _int, _i64, _i64, _i64, _i64, _int, C.c_float, _vp, _vp, _vp, _int, _vp],
    "strix_hc_mix_up": [_vp, _qv, _int, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _int, _vp],
    "strix_hc_inject_inv": [_vp, _vp, _vp, _i64, _i64, _i64, C.c_float, _vp, _int, _vp],
    "strix_to_chunk_major": [_int, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp],
    "strix_linear_q4_experts_gather": [_vp, _qv, _i64, _vp, _i64, _i64, _vp, _int, _vp, _vp],
    "strix_linear_q4_experts_combine": [_vp, _qv, _i64, _vp, _vp, _i64, _i64, _vp, _int, _vp, _vp],
    "strix_linear_q4_experts_gather_swiglu": [_vp, _qv, _i64, _vp, _i64, _i64, _vp, _int, _vp, _vp],
    "strix_linear_q5_experts_gather": [_vp, _qv, _i64, _vp, _i64, _i64, _vp, _int, _vp, _vp],
    "strix_linear_q5_experts_combine": [_vp, _qv, _i64, _vp, _vp, _i64, _i64, _vp, _int, _vp, _vp],
    "strix_linear_q5_experts_gather_swiglu": [_vp, _qv, _i64, _vp, _i64, _i64, _vp, _int, _vp, _vp],
    "strix_linear_qmix_experts_gather": [_vp, _qm, _vp, _i64, _i64, _vp, _int, _vp, _vp],
    "strix_linear_qmix_experts_combine": [_vp, _qm, _vp, _vp, _i64, _i64, _vp, _int, _vp, _vp],
    "strix_linear_qmix_experts_gather_swiglu": [_vp, _qm, _vp, _i64, _i64, _vp, _int, _vp, _vp],
    "strix_check_expert_error": [_vp, C.c_char_p],
    "strix_report_expert_error": [_vp, C.c_char_p],
    "strix_moe_route_workspace_bytes": [_i64, _i64, _i64],
    "strix_moe_group_routes": [_vp, _i64, _i64, _i64, _vp, _sz, _vp, _vp],
    "strix_linear_q4_experts_gather_grouped": [_vp, _qv, _i64, _vp, _sz, _i64, _i64, _vp, _int, _int, _vp],
    "strix_linear_q5_experts_gather_grouped": [_vp, _qv, _i64, _vp, _sz, _i64, _i64, _vp, _int, _int, _vp],
    "strix_linear_q4_experts_combine_grouped": [_vp, _qv, _i64, _vp, _vp, _vp, _sz, _vp, _i64, _i64, _vp, _int, _int, _vp],
    "strix_linear_q5_experts_combine_grouped": [_vp, _qv, _i64, _vp, _vp, _vp, _sz, _vp, _i64, _i64, _vp, _int, _int, _vp],
    "strix_linear_q4_experts_combine_grouped_fixed": [_vp, _qv, _i64, _vp, _vp, _vp, _sz, _i64, _i64, _vp, _int, _int, _vp],
    "strix_linear_qmix_experts_gather_grouped": [_vp, _qm, _vp, _sz, _i64, _i64, _vp, _int, _int, _vp],
    "strix_linear_qmix_experts_combine_grouped": [_vp, _qm, _vp, _vp, _vp, _sz, _vp, _i64, _i64, _vp, _int, _int, _vp],
    "strix_moe_combine_reduce": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _int, _vp],
    "strix_ep_meta_ints": [_i64, _i64],
    "strix_ep_plan_scratch_ints": [_i64],
    "strix_ep_plan": [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _int, _int, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp],
    "strix_ep_gather_rows": [_vp, _i64, _int, _vp, _vp, _int, _i64, _i64, _vp, _vp],
    "strix_ep_unpack": [_vp, _int, _i64, _i64, _vp, _vp, _vp],
    "strix_ep_row_sum": [_vp, _int, _vp, _int, _i64, _i64, _i64, _vp, _vp],
    "strix_ep_home_sum": [_vp, _int, _vp, _vp, _i64, _i64, _i64, _int, _i64, _i64, _vp, _int, _vp],
    "strix_ep_push_rows": [_vp, _i64, _int, _vp, _vp, _int, _int, _i64, _i64, _vp, _vp, _vp],
    "strix_ep_row_sum_push": [_vp, _int, _vp, _int, _int, _i64, _i64, _i64, _vp, _int, _vp],
    "strix_hash64": [_vp, _sz],
    "strix_umma_abort_count": [],
    "strix_workspace_refusal_count": [],
    "strix_umma_wait_cycles": [_vp, _int],
    "strix_last_error": [],
    "strix_version": [],
}
_RESTYPES = {
    "strix_row_bytes": _i64,
    "strix_ep_meta_ints": _i64,
    "strix_ep_plan_scratch_ints": _i64,
    "strix_hash64": C.c_uint64,
    "strix_umma_abort_count": C.c_uint,
    "strix_workspace_refusal_count": C.c_uint,
    "strix_umma_wait_cycles": None,
    "strix_moe_route_workspace_bytes": _sz,
    "strix_last_error": C.c_char_p,
    "strix_version": C.c_char_p,
}

for _name, _args in SIGNATURES.items():
    _f = getattr(lib, _name)  # AttributeError here = the library is stale: rebuild
    _f.argtypes = _args
    _f.restype = _RESTYPES.get(_name, _int)


def last_error():
    return lib.strix_last_error().decode("utf-8", "replace")


def call(name, *args):
    """Calls an int-returning entry point; raises StrixError with the library's message on failure."""
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise StrixError(last_error())
