"""ctypes binding of libhbsattn_b200.so (the C ABI of include/hbsattn_b200.h).

There is no fallback: if the shared library is missing or cannot be loaded the import of
this module raises, and every operator of the package fails with it.
"""
from __future__ import annotations

import ctypes
import os
import threading

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# HBSATTN_B200_LIBRARY selects another build of the same library (e.g. the strict-ordering build of build.py --strict).
LIB_PATH = os.environ.get("HBSATTN_B200_LIBRARY") or os.path.join(PKG_DIR, "libhbsattn_b200.so")

HBSA_DTYPE_BF16, HBSA_DTYPE_F16, HBSA_DTYPE_F32 = 0, 1, 2
HBSA_IMPL_AUTO, HBSA_IMPL_GENERIC, HBSA_IMPL_SM100 = 0, 1, 2
HBSA_STATUS_OK, HBSA_STATUS_BLOCK_COUNT_MISMATCH, HBSA_STATUS_WAIT_LIMIT = 0, 1, 2
STATUS_WORDS = 16

EXPORTED_SYMBOLS = (
    "hbsa_version",
    "hbsa_last_error",
    "hbsa_calculate_blocks",
    "hbsa_workspace_bytes",
    "hbsa_forward",
    "hbsa_build_schedule",
    "hbsa_attention",
    "hbsa_block_decisions",
    "hbsa_select_impl",
    "hbsa_backward",
    "hbsa_backward_workspace_bytes",
    "hbsa_read_status",
    "hbsa_forward_static_scratch",
    "hbsa_static_scratch_status",
    "hbsa_debug_set_wait_budget",
    "hbsa_debug_trace_bytes",
    "hbsa_debug_set_trace",
)
STATIC_SCRATCH_BYTES = 4 << 20


class ForwardArgs(ctypes.Structure):
    """Mirror of ``struct hbsa_forward_args``."""

    _fields_ = [
        ("struct_bytes", ctypes.c_size_t),
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
        ("q_stride", ctypes.c_int64 * 3),
        ("k_stride", ctypes.c_int64 * 3),
        ("v_stride", ctypes.c_int64 * 3),
        ("o_stride", ctypes.c_int64 * 3),
        ("cu_q_seqlens", ctypes.c_void_p),
        ("cu_k_seqlens", ctypes.c_void_p),
        ("block_mask", ctypes.c_void_p),
        ("mask_stride", ctypes.c_int64 * 3),
        ("total_q", ctypes.c_int32),
        ("total_k", ctypes.c_int32),
        ("nhead_q", ctypes.c_int32),
        ("nhead_k", ctypes.c_int32),
        ("headdim", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("num_q_block", ctypes.c_int32),
        ("num_k_block", ctypes.c_int32),
        ("q_block_size", ctypes.c_int32),
        ("k_block_size", ctypes.c_int32),
        ("causal", ctypes.c_int32),
        ("use_default_scale", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("dtype", ctypes.c_int32),
        ("impl", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("lse", ctypes.c_void_p),
        ("csr_row_ptr", ctypes.c_void_p),
        ("csr_col_idx", ctypes.c_void_p),
    ]


class BackwardArgs(ctypes.Structure):
    """Mirror of ``struct hbsa_backward_args``."""

    _fields_ = [
        ("struct_bytes", ctypes.c_size_t),
        ("fwd", ForwardArgs),
        ("d_o", ctypes.c_void_p),
        ("do_stride", ctypes.c_int64 * 3),
        ("dq", ctypes.c_void_p),
        ("dk", ctypes.c_void_p),
        ("dv", ctypes.c_void_p),
        ("grad_workspace", ctypes.c_void_p),
        ("grad_workspace_bytes", ctypes.c_size_t),
    ]


_lock = threading.Lock()
_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises if it is absent (no CPU or eager fallback exists)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python hbsattn_b200/build.py` "
                "(nvcc, sm_100a). hbsattn_b200 has no fallback path."
            )
        lib = ctypes.CDLL(LIB_PATH)
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        lib.hbsa_version.restype = i32
        lib.hbsa_version.argtypes = []
        lib.hbsa_last_error.restype = ctypes.c_char_p
        lib.hbsa_last_error.argtypes = []
        lib.hbsa_calculate_blocks.restype = i32
        lib.hbsa_calculate_blocks.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp]
        lib.hbsa_workspace_bytes.restype = ctypes.c_size_t
        lib.hbsa_workspace_bytes.argtypes = [i32, i32, i32, i32]
        lib.hbsa_forward.restype = i32
        lib.hbsa_forward.argtypes = [ctypes.POINTER(ForwardArgs), vp]
        for name in ("hbsa_build_schedule", "hbsa_attention"):
            getattr(lib, name).restype = i32
            getattr(lib, name).argtypes = [ctypes.POINTER(ForwardArgs), vp]
        lib.hbsa_block_decisions.restype = i32
        lib.hbsa_block_decisions.argtypes = [ctypes.POINTER(ForwardArgs), vp, vp, vp]
        lib.hbsa_backward.restype = i32
        lib.hbsa_backward.argtypes = [ctypes.POINTER(BackwardArgs), vp]
        lib.hbsa_backward_workspace_bytes.restype = ctypes.c_size_t
        lib.hbsa_backward_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64, i32, i32, i32]
        lib.hbsa_select_impl.restype = i32
        lib.hbsa_select_impl.argtypes = [ctypes.POINTER(ForwardArgs)]
        lib.hbsa_read_status.restype = i32
        lib.hbsa_read_status.argtypes = [vp, vp, vp]
        lib.hbsa_forward_static_scratch.restype = i32
        lib.hbsa_forward_static_scratch.argtypes = [ctypes.POINTER(ForwardArgs), vp]
        lib.hbsa_static_scratch_status.restype = i32
        lib.hbsa_static_scratch_status.argtypes = [vp, vp]
        lib.hbsa_debug_trace_bytes.restype = ctypes.c_size_t
        lib.hbsa_debug_trace_bytes.argtypes = []
        lib.hbsa_debug_set_trace.restype = None
        lib.hbsa_debug_set_trace.argtypes = [vp]
        lib.hbsa_debug_set_wait_budget.restype = None
        lib.hbsa_debug_set_wait_budget.argtypes = [ctypes.c_longlong, i32]
        if lib.hbsa_version() != 4:
            raise ImportError("libhbsattn_b200.so was built from a different ABI version")
        _lib = lib
        return lib


def last_error() -> str:
    return load().hbsa_last_error().decode("utf-8", "replace")
