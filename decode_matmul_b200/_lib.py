"""ctypes binding of libdmm.so: one Python function per entry point of include/dmm.h."""
from __future__ import annotations

import ctypes
import os

from . import build as _build

_LIB = None

# mirrors of the constants in include/dmm.h
SIGN_SLOW, SIGN_FAST = 0, 1
LAYOUT_TILE, LAYOUT_FAST = 0, 1
PATH_AUTO, PATH_GEMV, PATH_TCGEN05, PATH_TCGEN05_F8 = 0, 1, 2, 3
FLAG_ACCUMULATE, FLAG_PDL, FLAG_ATOMIC = 1, 2, 4
X_F16, X_F32, X_F32_SILU_MUL = 0, 1, 2
STATUS_WAIT_TIMEOUT, STATUS_BAD_CODEBOOK, STATUS_BAD_SMEM = 1, 2, 4

EXPORTS = (
    "dmm_i8", "dmm_f16", "dmm_f16_fused", "dmm_f16_fused_tp", "dmm_f16_tp_produce", "dmm_f16_tp_consume", "dmm_tp_finalize", "dmm_xrank_barrier", "dmm_xrank_allreduce_add", "dmm_f16_chain", "dmm_f16_noalloc", "dmm_decode", "dmm_workspace_bytes", "dmm_status", "dmm_select_path",
    "dmm_hint_next_weights", "dmm_set_wait_limit_ms", "dmm_launch_count", "dmm_error_string", "dmm_version",
)


CHAIN_MAX_OPS = 8


class ChainOp(ctypes.Structure):
    """``dmm_chain_op`` of include/dmm.h."""
    _fields_ = [("x", ctypes.c_void_p), ("x_kind", ctypes.c_int), ("x_ld", ctypes.c_int64), ("x_gap", ctypes.c_int64),
                ("codes", ctypes.c_void_p), ("scale", ctypes.c_float), ("out", ctypes.c_void_p), ("N", ctypes.c_int64),
                ("K", ctypes.c_int64), ("zero_ptr", ctypes.c_void_p), ("zero_count", ctypes.c_int64)]


def lib() -> ctypes.CDLL:
    """Loads the CUDA library, compiling it first when it is missing or stale and nvcc is at
    hand.  There is no fallback: without the library every operator raises."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _build.LIB
    try:
        path = _build.build()
    except Exception:
        if not os.path.exists(path):
            raise
    L = ctypes.CDLL(path)
    vp, i64, ci, cu, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t
    L.dmm_i8.argtypes = [vp, vp, vp, vp, i64, i64, i64, ci, ci, cu, vp, sz, vp]
    L.dmm_i8.restype = ci
    L.dmm_f16.argtypes = [vp, vp, vp, ctypes.c_float, vp, i64, i64, i64, ci, ci, ci, cu, vp, sz, vp]
    L.dmm_f16.restype = ci
    L.dmm_f16_fused.argtypes = [vp, ci, i64, i64, vp, vp, ctypes.c_float, vp, i64, i64, i64, ci, ci, ci, cu, vp, i64, vp, sz,
                                vp]
    L.dmm_f16_fused.restype = ci
    L.dmm_f16_fused_tp.argtypes = [vp, ci, i64, i64, vp, vp, ctypes.c_float, vp, ci, i64, i64, i64, ci, cu, vp, i64, vp, vp,
                                   i64, vp]
    L.dmm_f16_fused_tp.restype = ci
    L.dmm_f16_tp_produce.argtypes = [vp, ci, i64, i64, vp, vp, ctypes.c_float, vp, vp, ci, ci, i64, i64, i64, ci, cu, vp]
    L.dmm_f16_tp_produce.restype = ci
    L.dmm_f16_tp_consume.argtypes = [vp, vp, i64, vp, vp, ci, i64, vp, vp, ctypes.c_float, vp, i64, i64, i64, ci, cu, vp, i64, vp]
    L.dmm_f16_tp_consume.restype = ci
    L.dmm_tp_finalize.argtypes = [vp, vp, vp, vp, ci, i64, vp]
    L.dmm_tp_finalize.restype = ci
    L.dmm_xrank_barrier.argtypes = [vp, ci, ci, vp]
    L.dmm_xrank_barrier.restype = ci
    L.dmm_xrank_allreduce_add.argtypes = [vp, vp, vp, i64, vp, ci, ci, vp]
    L.dmm_xrank_allreduce_add.restype = ci
    L.dmm_f16_chain.argtypes = [vp, ci, vp, i64, ci, cu, vp]
    L.dmm_f16_chain.restype = ci
    L.dmm_f16_noalloc.argtypes = [vp, vp, vp, ctypes.c_float, vp, i64, i64, i64, ci, cu, vp]
    L.dmm_f16_noalloc.restype = ci
    L.dmm_decode.argtypes = [vp, vp, ci, vp, i64, i64, ci, ci, vp]
    L.dmm_decode.restype = ci
    L.dmm_workspace_bytes.argtypes = [i64, i64, i64]
    L.dmm_workspace_bytes.restype = sz
    L.dmm_status.argtypes = [ctypes.POINTER(cu)]
    L.dmm_status.restype = ci
    L.dmm_select_path.argtypes = [i64, i64, i64]
    L.dmm_select_path.restype = ci
    L.dmm_hint_next_weights.argtypes = [vp, i64, i64]
    L.dmm_hint_next_weights.restype = ci
    L.dmm_set_wait_limit_ms.argtypes = [cu]
    L.dmm_set_wait_limit_ms.restype = ci
    L.dmm_launch_count.argtypes = []
    L.dmm_launch_count.restype = ctypes.c_uint64
    L.dmm_error_string.argtypes = [ci]
    L.dmm_error_string.restype = ctypes.c_char_p
    L.dmm_version.argtypes = []
    L.dmm_version.restype = ctypes.c_char_p
    _LIB = L
    return L


def check(rc: int, what: str) -> None:
    """Turns a non-zero return value into RuntimeError, as TORCH_CHECK does in the
    reference's host wrappers (decode_matmul_cuda.cu:186-207)."""
    if rc != 0:
        msg = lib().dmm_error_string(rc).decode()
        raise RuntimeError(f"{what}: {msg} (code {rc})")
