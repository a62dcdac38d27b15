"""ctypes binding of libspsattn.so (the C ABI declared in include/spsattn.h).

There is no fallback: if the shared library is missing or fails to load, every
entry point raises.  Build it with ``python -m sps_b200.build``.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libspsattn.so")

DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2
PARITY_EVEN, PARITY_ODD, PARITY_NONE = 0, 1, -1
NO_WINDOW = -2147483648
NOALLOC_SCRATCH_BYTES = 16 << 20
FLAG_PERSISTENT_Q_SKIPS_TEMPORARY = 1

EXPORTS = (
    "spsattn_version", "spsattn_strerror",
    "spsattn_prefill_workspace_bytes", "spsattn_prefill_fwd", "spsattn_prefill_fwd_strided",
    "spsattn_decode_workspace_bytes", "spsattn_decode_fwd", "spsattn_decode_fwd_noalloc",
    "spsattn_kv_update", "spsattn_fill_decode_caches", "spsattn_rope_cast", "spsattn_debug_visibility",
    "spsattn_decode_step_workspace_bytes", "spsattn_decode_step", "spsattn_qkv_rope_cast",
    "spsattn_add_rmsnorm", "spsattn_swiglu", "spsattn_debug_decode_path", "spsattn_debug_prefill_path", "spsattn_debug_wait_expiry",
    "spsattn_prefill_bwd_workspace_bytes", "spsattn_prefill_bwd", "spsattn_prefill_bwd_strided",
)


class Segment(C.Structure):
    """struct spsattn_segment"""
    _fields_ = [
        ("k", C.c_void_p), ("v", C.c_void_p), ("seq_offset", C.c_void_p),
        ("seq_stride", C.c_int64), ("head_stride", C.c_int64), ("row_stride", C.c_int64),
        ("lengths", C.c_void_p), ("lengths_per_head", C.c_int32), ("max_rows", C.c_int32),
        ("query_mask", C.c_uint32), ("reserved", C.c_uint32),
    ]


class Extra(C.Structure):
    """struct spsattn_extra"""
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("query_mask", C.c_uint32),
                ("reserved", C.c_uint32)]


class KvAppend(C.Structure):
    """struct spsattn_kv_append"""
    _fields_ = [
        ("nw_k", C.c_void_p), ("nw_v", C.c_void_p), ("nw_len", C.c_void_p), ("nw_pos", C.c_void_p),
        ("br_k", C.c_void_p), ("br_v", C.c_void_p), ("br_len", C.c_void_p),
        ("k_window", C.c_void_p), ("v_window", C.c_void_p),
        ("k_retained", C.c_void_p), ("v_retained", C.c_void_p), ("active", C.c_void_p),
        ("window_storage", C.c_int32), ("retained_storage", C.c_int32),
        ("window_tokens", C.c_int32), ("reserved", C.c_int32),
    ]


class RopeGroup(C.Structure):
    """struct spsattn_rope_group"""
    _fields_ = [("out", C.c_void_p), ("stride_b", C.c_int64), ("stride_n", C.c_int64),
                ("stride_h", C.c_int64), ("rotate", C.c_int32), ("reserved", C.c_int32)]


class SpsAttnError(RuntimeError):
    pass


_lib = None


def load() -> C.CDLL:
    """Load the shared library once and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise SpsAttnError(
            f"{LIB_PATH} is missing: the CUDA extension is required (python -m sps_b200.build); "
            "there is no CPU or PyTorch fallback")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, f32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
    lib.spsattn_version.restype = i32
    lib.spsattn_strerror.restype = C.c_char_p
    lib.spsattn_strerror.argtypes = [i32]
    lib.spsattn_prefill_workspace_bytes.restype = sz
    lib.spsattn_prefill_workspace_bytes.argtypes = [i32, i32, i32, i32]
    lib.spsattn_prefill_fwd.restype = i32
    lib.spsattn_prefill_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i32, i64, i64, i32, i32, i32, i32, i32,
                                        f32, i32, i32, i32, i32, vp, sz, vp, vp]
    lib.spsattn_prefill_bwd_workspace_bytes.restype = sz
    lib.spsattn_prefill_bwd_workspace_bytes.argtypes = [i32, i32, i32, i32]
    lib.spsattn_prefill_bwd.restype = i32
    lib.spsattn_prefill_bwd.argtypes = [vp] * 10 + [i32, i64, i64, i32, i32, i32, i32, i32, f32,
                                                     i32, i32, i32, i32, vp, sz, vp, vp]
    p64 = C.POINTER(C.c_int64)
    lib.spsattn_prefill_bwd_strided.restype = i32
    lib.spsattn_prefill_bwd_strided.argtypes = [vp] * 9 + [p64, vp, i32, i64, i64, i32, i32, i32, i32, i32, f32,
                                                           i32, i32, i32, i32, vp, sz, vp, vp]
    lib.spsattn_prefill_fwd_strided.restype = i32
    lib.spsattn_prefill_fwd_strided.argtypes = [vp, vp, vp, vp, vp, p64, p64, p64, p64, vp, i32, i64, i64,
                                                i32, i32, i32, i32, i32, f32, i32, i32, i32, i32, vp, sz, vp, vp]
    lib.spsattn_decode_workspace_bytes.restype = sz
    lib.spsattn_decode_workspace_bytes.argtypes = [i32, i32, i32, i32, C.POINTER(Segment), i32]
    lib.spsattn_decode_fwd.restype = i32
    lib.spsattn_decode_fwd.argtypes = [vp, i32, vp, C.POINTER(Segment), i32, C.POINTER(Extra), i32,
                                       i32, i32, i32, i32, f32, vp, sz, vp, vp]
    lib.spsattn_decode_fwd_noalloc.restype = i32
    lib.spsattn_decode_fwd_noalloc.argtypes = [vp, i32, vp, C.POINTER(Segment), i32, C.POINTER(Extra), i32,
                                               i32, i32, i32, i32, f32, vp, vp]
    lib.spsattn_kv_update.restype = i32
    lib.spsattn_kv_update.argtypes = [vp] * 12 + [i32] * 7 + [vp]
    lib.spsattn_fill_decode_caches.restype = i32
    lib.spsattn_fill_decode_caches.argtypes = [vp, vp, i64, i64, i64, vp, vp, vp, vp, vp, vp, vp, vp,
                                               i32, i32, i32, i32, i32, i32, i32, i32, i32, vp]
    lib.spsattn_rope_cast.restype = i32
    lib.spsattn_rope_cast.argtypes = [vp, i32, i64, i64, i64, vp, i64, vp, i32, i64, i64, i64,
                                      i32, i32, i32, i32, i32, vp]
    lib.spsattn_decode_step_workspace_bytes.restype = sz
    lib.spsattn_decode_step_workspace_bytes.argtypes = [i32, i32, i32, i32, C.POINTER(Segment), i32]
    lib.spsattn_decode_step.restype = i32
    lib.spsattn_decode_step.argtypes = [vp, i32, vp, i32, C.POINTER(Segment), i32, C.POINTER(Extra), i32,
                                        C.POINTER(KvAppend), i32, i32, i32, i32, f32, vp, sz, vp, vp]
    lib.spsattn_qkv_rope_cast.restype = i32
    lib.spsattn_qkv_rope_cast.argtypes = [vp, i32, i64, i64, i64, vp, i64, C.POINTER(RopeGroup), i32, i32,
                                          i32, i32, i32, i32, vp]
    lib.spsattn_add_rmsnorm.restype = i32
    lib.spsattn_add_rmsnorm.argtypes = [vp, vp, vp, vp, i32, C.c_longlong, i32, f32, vp]
    lib.spsattn_swiglu.restype = i32
    lib.spsattn_swiglu.argtypes = [vp, vp, i32, C.c_longlong, i32, vp]
    lib.spsattn_debug_decode_path.restype = i32
    lib.spsattn_debug_decode_path.argtypes = [i32]
    lib.spsattn_debug_wait_expiry.restype = i32
    lib.spsattn_debug_wait_expiry.argtypes = [vp, C.c_ulonglong, vp, vp]
    lib.spsattn_debug_prefill_path.restype = i32
    lib.spsattn_debug_prefill_path.argtypes = [i32]
    lib.spsattn_debug_visibility.restype = i32
    lib.spsattn_debug_visibility.argtypes = [vp, vp, i32, i64, i64, i32, i32, i32, i32, i32, i32, vp, sz, vp]
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().spsattn_strerror(code).decode()
        raise SpsAttnError(f"{what} failed: {msg} (code {code})")
