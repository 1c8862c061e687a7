"""ctypes binding of the C-ABI library (include/deltanet_b200.h).

The library is the product: if it cannot be loaded this module raises, there is no
fallback of any kind.  Build it with ``deltanet-tpu_b200/csrc/build.sh``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# DELTANET_B200_LIB points at another build of the same library (a debug or instrumented one)
LIB_PATH = os.environ.get("DELTANET_B200_LIB") or os.path.join(_HERE, "libdeltanet_b200.so")

DN_F32, DN_BF16 = 0, 1
DN_PREC_FP32, DN_PREC_BF16 = 0, 1
DN_QK_L2NORM = 1 << 0
DN_FUSE_PROLOGUE = 1 << 1
DN_HAS_INIT = 1 << 2
DN_STABILITY_GUARD = 1 << 3
DN_STATE_FP32_MM = 1 << 4
DN_INFERENCE = 1 << 5
DN_TRUNC_DT_BF16 = 1 << 6
DN_RESET_PER_HEAD = 1 << 7
DN_SP_SKIP_PROVISIONAL = 1 << 8


class Shape(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "B", "L", "Hk", "Hv", "K", "V", "chunk", "g_heads", "g_cols", "b_heads", "b_cols",
        "w_heads", "w_cols", "qkv_dtype", "gate_dtype", "precision")] + [
        ("flags", C.c_uint32), ("scale", C.c_float)]


class Exec(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("H", "Vw", "G", "NC", "pre_dtype", "chunk")]


class Residuals(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("W", "U", "M", "qe", "ke", "lam_end", "T", "states")]


class DecodeShape(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "B", "Hk", "Hv", "K", "V", "g_heads", "g_cols", "b_heads", "b_cols", "w_heads", "w_cols",
        "qkv_dtype", "gate_dtype", "state_in_dtype", "state_out_dtype")] + [
        ("flags", C.c_uint32), ("scale", C.c_float), ("stability_tau", C.c_float)]


_P = C.c_void_p
_SIGNATURES = {
    "dn_version": (C.c_int, []),
    "dn_device_error": (C.c_int, []),
    "dn_device_error_reset": (None, []),
    "dn_cap_state": (C.c_int, [_P, C.c_int64, C.c_int32, C.c_int32, C.c_float, _P]),
    "dn_status_string": (C.c_char_p, [C.c_int]),
    "dn_exec_view": (C.c_int, [C.POINTER(Shape), C.POINTER(Exec)]),
    "dn_residual_bytes": (C.c_size_t, [C.POINTER(Shape)]),
    "dn_residual_carve": (C.c_int, [C.POINTER(Shape), _P, C.POINTER(Residuals)]),
    "dn_scratch_bytes": (C.c_size_t, [C.POINTER(Shape), C.c_int, C.c_int]),
    "dn_canonical_segments": (C.c_int, [_P, _P, _P, C.c_int32, C.c_int32, _P]),
    "dn_cu_seqlens_segments": (C.c_int, [_P, C.c_int32, _P, _P, C.c_int32, C.c_int32, _P]),
    "dn_chunk_fwd": (C.c_int, [C.POINTER(Shape)] + [_P] * 10 + [C.POINTER(Residuals), _P, C.c_size_t, _P]),
    "dn_chunk_bwd": (C.c_int, [C.POINTER(Shape)] + [_P] * 8 + [C.POINTER(Residuals)] + [_P] * 9 + [_P, C.c_size_t, _P]),
    "dn_prepass_fwd": (C.c_int, [C.POINTER(Shape)] + [_P] * 7 + [C.POINTER(Residuals), _P, C.c_size_t, _P]),
    "dn_state_fwd": (C.c_int, [C.POINTER(Shape), C.POINTER(Residuals)] + [_P] * 5),
    "dn_recompute_states": (C.c_int, [C.POINTER(Shape), C.POINTER(Residuals)] + [_P] * 3),
    "dn_state_bwd": (C.c_int, [C.POINTER(Shape), C.POINTER(Residuals)] + [_P] * 7),
    "dn_prepass_bwd": (C.c_int, [C.POINTER(Shape)] + [_P] * 7 + [C.POINTER(Residuals)] + [_P] * 9 + [_P, C.c_size_t, _P]),
    "dn_decode_step": (C.c_int, [C.POINTER(DecodeShape)] + [_P] * 11),
    "dn_sp_transition": (C.c_int, [C.POINTER(Shape), C.POINTER(Residuals)] + [_P] * 4),
    "dn_sp_summary": (C.c_int, [C.POINTER(Shape), C.POINTER(Residuals)] + [_P] * 5),
    "dn_sp_correct_fwd": (C.c_int, [C.POINTER(Shape), C.POINTER(Residuals)] + [_P] * 4),
    "dn_sp_correct_bwd": (C.c_int, [C.POINTER(Shape), C.POINTER(Residuals)] + [_P] * 6),
    "dn_sp_apply": (C.c_int, [_P] * 5 + [C.c_int32] * 6 + [_P]),
    "dn_gdn_producer_scratch_bytes": (C.c_size_t, [C.c_int32] * 4),
    "dn_gdn_producer_fwd": (C.c_int, [_P] * 4 + [C.c_int32] * 8 + [_P] * 4),
    "dn_gdn_producer_bwd": (C.c_int, [_P] * 4 + [C.c_int32] * 8 + [_P] * 7 + [C.c_size_t, _P]),
    "dn_gdn_gates_fwd": (C.c_int, [_P] * 4 + [C.c_int32] * 4 + [_P] * 3),
    "dn_gdn_gates_bwd": (C.c_int, [_P] * 6 + [C.c_int32] * 4 + [_P] * 5),
    "dn_gated_rmsnorm_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "dn_gated_rmsnorm_fwd": (C.c_int, [_P] * 3 + [C.c_int64, C.c_int32, C.c_int32, C.c_float, _P, _P]),
    "dn_gated_rmsnorm_bwd": (C.c_int, [_P] * 3 + [C.c_int64, C.c_int32, C.c_int32, C.c_float] + [_P] * 5 + [C.c_size_t, _P]),
    "dn_static_scratch_bytes": (C.c_size_t, []),
    "dn_prepass_fwd_static": (C.c_int, [C.POINTER(Shape)] + [_P] * 7 + [C.POINTER(Residuals), _P]),
    "dn_selftest_umma": (C.c_int, [C.c_int32] * 4 + [_P] * 5),
    "dn_launches_total": (C.c_int64, []),
    "dn_launch_count": (C.c_int, [C.POINTER(Shape), C.c_int, C.c_int]),
}
EXPORTED = tuple(_SIGNATURES)

_lib = None


def lib():
    """The loaded library; raises (never falls back) if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"deltanet_b200: the CUDA library {LIB_PATH} is missing; build it with "
                "deltanet-tpu_b200/csrc/build.sh (there is no CPU or eager fallback).")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int, what: str):
    if status != 0:
        raise RuntimeError(f"deltanet_b200: {what} failed: {lib().dn_status_string(status).decode()} (status {status})")
