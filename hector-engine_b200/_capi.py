"""ctypes binding of libhkv's C ABI (include/hkv.h).

There is no fallback: if the shared library is missing or cannot be loaded this module
raises, and every call that needs a GPU fails with the library's own status code.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libhkv.so")

HKV_OK = 0
STATUS_NAMES = {
    0: "HKV_OK", 1: "HKV_ERR_INVALID_ARG", 2: "HKV_ERR_GEOMETRY", 3: "HKV_ERR_ALIGNMENT",
    4: "HKV_ERR_CUDA", 5: "HKV_ERR_NO_DEVICE", 6: "HKV_ERR_WORKSPACE", 7: "HKV_ERR_TOO_LARGE",
    8: "HKV_ERR_DEVICE_FAULT",
}
LAYOUT_LINEAR, LAYOUT_RING = 0, 1
FLAG_SCALAR_POSITION, FLAG_APPEND_ONLY = 1, 2
ABI_VERSION = 2
KERNEL_AUTO, KERNEL_GENERIC, KERNEL_TMA = 0, 1, 2


class HkvGeometry(C.Structure):
    """Mirror of `struct hkv_geometry` (include/hkv.h)."""
    _fields_ = [
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("slots", C.c_int32), ("window_size", C.c_int32),
        ("layout", C.c_int32), ("chunk_tiles", C.c_int32), ("batch_stride_elems", C.c_int64),
        ("shard_rank", C.c_int32), ("shard_count", C.c_int32), ("shard_block", C.c_int32),
        ("kernel_select", C.c_int32), ("max_seq_new", C.c_int32), ("flags", C.c_int32),
        ("tune_prefill_splits", C.c_int32), ("tune_prefill_kernel", C.c_int32), ("tune_tma_groups", C.c_int32),
        ("q_seq_stride_elems", C.c_int32), ("new_kv_seq_stride_elems", C.c_int32), ("reserved", C.c_int32 * 1),
    ]


MAX_PEERS = 8


class HkvExchange(C.Structure):
    """Mirror of `struct hkv_exchange` (include/hkv.h): the mailboxes of a peer exchange."""
    _fields_ = [
        ("rank", C.c_int32), ("world", C.c_int32), ("mailbox", C.c_void_p * MAX_PEERS),
        ("wait_limit_ms", C.c_int32), ("reserved", C.c_int32),
    ]


# name -> (restype, argtypes); every symbol include/hkv.h declares
_VP, _I32P, _F32P = C.c_void_p, C.c_void_p, C.c_void_p
SIGNATURES = {
    "hkv_abi_version": (C.c_int, []),
    "hkv_status_string": (C.c_char_p, [C.c_int]),
    "hkv_ctx_create": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(HkvGeometry)]),
    "hkv_ctx_destroy": (C.c_int, [_VP]),
    "hkv_ctx_last_error": (C.c_char_p, [_VP]),
    "hkv_workspace_bytes": (C.c_size_t, [C.POINTER(HkvGeometry)]),
    "hkv_ctx_device_status": (C.c_int, [_VP, _VP, C.POINTER(C.c_int32)]),
    "hkv_ctx_kernel": (C.c_int, [_VP]),
    "hkv_ctx_launches_per_decode": (C.c_int, [_VP]),
    "hkv_append": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _I32P, C.c_int32, _VP]),
    "hkv_append_at": (C.c_int, [_VP, _VP, _VP, _VP, _VP, C.c_int32, C.c_int32, _VP]),
    "hkv_decode_attention": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _I32P, C.c_float, _VP]),
    "hkv_decode_attention_len": (C.c_int, [_VP, _VP, _VP, _VP, _VP, C.c_int32, C.c_float, _VP]),
    "hkv_append_decode_attention": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I32P, C.c_float, _VP]),
    "hkv_decode_attention_static": (C.c_int, [C.POINTER(HkvGeometry), _VP, _VP, _VP, _VP, _I32P, C.c_float, _VP]),
    "hkv_prefill_attention": (C.c_int, [_VP, _VP, _VP, _VP, _VP, C.c_int32, C.c_int32, C.c_float, _VP]),
    "hkv_prefill_append_attention": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, C.c_int32, C.c_int32, C.c_float, _VP]),
    "hkv_partial_floats": (C.c_size_t, [C.POINTER(HkvGeometry)]),
    "hkv_decode_partials": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, _F32P, _I32P, C.c_float, _VP]),
    "hkv_combine_partials": (C.c_int, [_VP, _F32P, C.c_int32, _VP, _VP]),
    "hkv_exchange_bytes": (C.c_int, [_VP, C.c_int32, C.POINTER(C.c_size_t)]),
    "hkv_decode_partials_publish": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, C.POINTER(HkvExchange), _I32P, C.c_float, _VP]),
    "hkv_merge_published": (C.c_int, [_VP, C.POINTER(HkvExchange), _VP, _VP]),
    "hkv_append_decode_attention_host": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I32P, C.c_float, _VP]),
    "hkv_append_decode_attention_host_pipelined": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I32P, C.c_float, _VP]),
    "hkv_host_flush": (C.c_int, [_VP, _VP]),
    "hkv_qk_norm_rope_kv": (C.c_int, [_VP] * 8 + [_I32P, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_float, C.c_float, _VP]),
    "hkv_ctx_selftest_bounded_wait": (C.c_int, [_VP, C.c_int32, _VP]),
    "hkv_ctx_profile_begin": (C.c_int, [_VP, C.c_int32]),
    "hkv_ctx_profile_end": (C.c_int, [_VP, _VP, C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_int32)]),
    "hkv_slot_of_position": (C.c_int32, [C.POINTER(HkvGeometry), C.c_int32]),
    "hkv_position_of_slot": (C.c_int32, [C.POINTER(HkvGeometry), C.c_int32, C.c_int32]),
    "hkv_plan_decode_tiles": (C.c_int, [C.POINTER(HkvGeometry), C.c_int32] + [C.POINTER(C.c_int32)] * 3),
    "hkv_plan_decode_spans": (C.c_int, [C.POINTER(HkvGeometry), C.c_void_p, C.c_int32] + [C.c_void_p] * 2 + [C.POINTER(C.c_int32)] * 2),
    "hkv_plan_sequence": (C.c_int, [C.POINTER(HkvGeometry), C.c_int32, C.c_int32] + [C.POINTER(C.c_int32)] * 4),
    "hkv_plan_prefill": (C.c_int, [C.POINTER(HkvGeometry), C.c_int32, C.c_int32, C.c_int32] + [C.POINTER(C.c_int32)] * 4),
    "hkv_preferred_prefill_chunk": (C.c_int32, [C.POINTER(HkvGeometry), C.c_int32, C.c_int32]),
    "hkv_fill_synthetic": (C.c_int, [_VP, C.c_uint64, C.c_uint64, C.c_uint64, _VP]),
}

_lib = None


def load() -> C.CDLL:
    """Loads libhkv.so (once). Raises if it was not built — there is no other path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python hector-engine_b200/build.py` "
            "(needs nvcc); this package has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class HkvError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
