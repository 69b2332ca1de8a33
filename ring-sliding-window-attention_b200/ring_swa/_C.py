"""ctypes binding of librswa.so (the C ABI declared in include/rswa.h).

There is no fallback: if the library is missing or a call is rejected, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librswa.so")

RSWA_MAX_SPANS = 10
TILE = 128
DTYPE_BF16, DTYPE_FP16, DTYPE_F32 = 0, 1, 2
BWD_INIT, BWD_FINISH = 1, 2


class Span(C.Structure):
    _fields_ = [
        ("k", C.c_void_p), ("v", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("kv_stride_b", C.c_int64), ("kv_stride_t", C.c_int64), ("kv_stride_h", C.c_int64),
        ("dkv_stride_b", C.c_int64), ("dkv_stride_t", C.c_int64), ("dkv_stride_h", C.c_int64),
        ("pos_start", C.c_int32), ("len", C.c_int32), ("grad_fp32", C.c_int32), ("reserved", C.c_int32),
    ]


class Geom(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("batch", C.c_int32), ("q_len", C.c_int32), ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("q_pos_start", C.c_int32), ("window", C.c_int32), ("n_sink", C.c_int32),
        ("softmax_scale", C.c_float),
        ("cu_seqlens", C.c_void_p), ("n_seqs", C.c_int32), ("n_spans", C.c_int32),
        ("spans", Span * RSWA_MAX_SPANS),
    ]


class FwdParams(C.Structure):
    _fields_ = [
        ("g", Geom),
        ("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_t", C.c_int64), ("q_stride_h", C.c_int64),
        ("out", C.c_void_p), ("o_stride_b", C.c_int64), ("o_stride_t", C.c_int64), ("o_stride_h", C.c_int64),
        ("lse", C.c_void_p), ("lse_stride_b", C.c_int64), ("lse_stride_h", C.c_int64),
        ("q_tile_begin", C.c_int32), ("q_tile_end", C.c_int32),
        ("status", C.c_void_p),
        ("carry", C.c_int32), ("reserved", C.c_int32),
    ]


class BwdParams(C.Structure):
    _fields_ = [
        ("g", Geom),
        ("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_t", C.c_int64), ("q_stride_h", C.c_int64),
        ("out", C.c_void_p), ("o_stride_b", C.c_int64), ("o_stride_t", C.c_int64), ("o_stride_h", C.c_int64),
        ("dout", C.c_void_p), ("do_stride_b", C.c_int64), ("do_stride_t", C.c_int64), ("do_stride_h", C.c_int64),
        ("lse", C.c_void_p), ("lse_stride_b", C.c_int64), ("lse_stride_h", C.c_int64),
        ("dq", C.c_void_p), ("dq_stride_b", C.c_int64), ("dq_stride_t", C.c_int64), ("dq_stride_h", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("flags", C.c_int32),
        ("status", C.c_void_p),
        ("ev_main_start", C.c_void_p), ("ev_main_stop", C.c_void_p), ("ev_main_mid", C.c_void_p),
    ]


class MergeParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("batch", C.c_int32), ("q_len", C.c_int32), ("n_heads", C.c_int32), ("head_dim", C.c_int32),
        ("o_a", C.c_void_p), ("o_b", C.c_void_p), ("o", C.c_void_p),
        ("oa_stride_b", C.c_int64), ("oa_stride_t", C.c_int64), ("oa_stride_h", C.c_int64),
        ("ob_stride_b", C.c_int64), ("ob_stride_t", C.c_int64), ("ob_stride_h", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_t", C.c_int64), ("o_stride_h", C.c_int64),
        ("lse_a", C.c_void_p), ("lse_b", C.c_void_p), ("lse", C.c_void_p),
        ("lse_stride_b", C.c_int64), ("lse_stride_h", C.c_int64),
    ]


class MergeAccParams(C.Structure):
    _fields_ = [
        ("new_dtype", C.c_int32), ("lse_f64", C.c_int32),
        ("batch", C.c_int32), ("q_len", C.c_int32), ("n_heads", C.c_int32), ("head_dim", C.c_int32),
        ("acc_o", C.c_void_p), ("acc_stride_b", C.c_int64), ("acc_stride_t", C.c_int64), ("acc_stride_h", C.c_int64),
        ("new_o", C.c_void_p), ("new_stride_b", C.c_int64), ("new_stride_t", C.c_int64), ("new_stride_h", C.c_int64),
        ("acc_lse", C.c_void_p), ("acc_lse_stride_b", C.c_int64), ("acc_lse_stride_h", C.c_int64),
        ("new_lse", C.c_void_p), ("new_lse_stride_b", C.c_int64), ("new_lse_stride_h", C.c_int64),
    ]


# every symbol include/rswa.h declares, with its signature
SYMBOLS = {
    "rswa_abi_version": (C.c_int, []),
    "rswa_last_error": (C.c_char_p, []),
    "rswa_fwd": (C.c_int, [C.POINTER(FwdParams), C.c_void_p]),
    "rswa_bwd_workspace_bytes": (C.c_int64, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "rswa_bwd": (C.c_int, [C.POINTER(BwdParams), C.c_void_p]),
    "rswa_bwd_noalloc": (C.c_int, [C.POINTER(BwdParams), C.c_void_p]),
    "rswa_noalloc_scratch_bytes": (C.c_int64, []),
    "rswa_merge": (C.c_int, [C.POINTER(MergeParams), C.c_void_p]),
    "rswa_merge_acc": (C.c_int, [C.POINTER(MergeAccParams), C.c_void_p]),
    "rswa_halo_accumulate": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                       C.c_int64, C.c_void_p]),
    "rswa_halo_accumulate_cast": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                            C.c_int32, C.c_int32, C.c_int64, C.c_void_p]),
    "rswa_cast_from_f32": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                     C.c_int64, C.c_void_p]),
    "rswa_peer_put": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int32,
                                C.c_void_p]),
    "rswa_flag_set": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "rswa_flag_wait": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int64, C.c_void_p]),
    "rswa_event_create": (C.c_void_p, []),
    "rswa_event_destroy": (None, [C.c_void_p]),
    "rswa_event_record": (C.c_int, [C.c_void_p, C.c_void_p]),
    "rswa_event_wait": (C.c_int, [C.c_void_p, C.c_void_p]),
    "rswa_event_elapsed_ms": (C.c_float, [C.c_void_p, C.c_void_p]),
    "rswa_selftest_mma": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """Loads librswa.so once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python ring-sliding-window-attention_b200/build.py` "
                "(needs nvcc with sm_100a support). There is no fallback path."
            )
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        if handle.rswa_abi_version() != 1:
            raise ImportError("librswa.so ABI version mismatch; rebuild it")
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    """Maps a negative return code to the exception the reference's asserts would raise."""
    if rc == 0:
        return
    msg = lib().rswa_last_error().decode("utf-8", "replace")
    if rc in (-1, -2, -4):
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg} (code {rc})")
