"""ctypes loader for the CPU oracle (oracle/hkv_oracle.cpp) and, when present, for the
reference's own kernels rebuilt for sm_100a (oracle/_ref).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the benchmark's
CPU-baseline / reference legs. The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_LIB = os.path.join(HERE, "_build", "libhkv_oracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libhector_ref_attention.so")

_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    src = os.path.join(HERE, "hkv_oracle.cpp")
    if not os.path.exists(ORACLE_LIB) or os.path.getmtime(ORACLE_LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    lib = C.CDLL(ORACLE_LIB)
    lib.hkv_oracle_hardware_threads.restype = C.c_int
    lib.hkv_oracle_f2h.restype = C.c_uint16
    lib.hkv_oracle_f2h.argtypes = [C.c_float]
    lib.hkv_oracle_h2f.restype = C.c_float
    lib.hkv_oracle_h2f.argtypes = [C.c_uint16]
    lib.hkv_oracle_fill.argtypes = [_u16p, C.c_uint64, C.c_uint64, C.c_uint64]
    lib.hkv_oracle_append.argtypes = [_u16p, _u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int,
                                      C.c_int, C.c_int64, _i32p, C.c_int]
    lib.hkv_oracle_decode.argtypes = [_u16p, _u16p, _u16p, _u16p, C.c_void_p, C.c_int, _i32p, C.c_int,
                                      C.c_int, C.c_int, C.c_int, C.c_int64, C.c_float, C.c_int,
                                      C.c_int, C.c_int, C.c_int]
    lib.hkv_oracle_prefill.argtypes = [_u16p, _u16p, _u16p, _u16p, C.c_void_p, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int,
                                       C.c_int, C.c_int, C.c_int]
    lib.hkv_oracle_qk_norm_rope.argtypes = [_u16p, _u16p, C.c_void_p, _u16p, _u16p, C.c_void_p, C.c_void_p,
                                            C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _i32p,
                                            C.c_int, C.c_int, C.c_float, C.c_float, C.c_float]
    lib.hkv_oracle_gemma4_layout.restype = C.c_int64
    lib.hkv_oracle_gemma4_layout.argtypes = [C.c_int, C.c_int, _i32p, _i32p, C.c_int, C.c_int, C.c_int,
                                             C.c_int, _i32p, _i64p, _i32p]
    _lib = lib
    return lib


def hardware_threads() -> int:
    return load().hkv_oracle_hardware_threads()


def as_u16(a) -> np.ndarray:
    """fp16 ndarray -> contiguous uint16 view (no copy when already contiguous)."""
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == np.float16 else a.astype(np.uint16, copy=False)


def fill(seed: int, first_index: int, count: int) -> np.ndarray:
    """Synthetic fp16 stream (same bits as hkv_fill_synthetic on the GPU)."""
    out = np.empty(count, dtype=np.uint16)
    load().hkv_oracle_fill(out, seed & 0xFFFFFFFFFFFFFFFF, first_index, count)
    return out.view(np.float16)


def append(new_k, new_v, k_cache, v_cache, pos, layout=0, batch_stride=0):
    """In-place append into k_cache/v_cache ([B, slots, KVH, HD] fp16 arrays)."""
    B, S, KVH, HD = new_k.shape
    slots = k_cache.shape[1]
    kc, vc = as_u16(k_cache), as_u16(v_cache)
    assert kc.base is k_cache or kc is k_cache or np.shares_memory(kc, k_cache)
    load().hkv_oracle_append(as_u16(new_k), as_u16(new_v), kc, vc, B, S, KVH, HD, slots, batch_stride,
                             np.ascontiguousarray(pos, dtype=np.int32), layout)


def decode(q, k_cache, v_cache, total, scale, window=0, layout=0, mode=0, threads=1,
           return_f32=False):
    """q [B, H, HD] (or [B,1,H,HD]); planes [B, slots, KVH, HD]; total int32[B]."""
    q = np.ascontiguousarray(q).reshape(q.shape[0], -1, q.shape[-1])
    B, H, HD = q.shape
    slots, KVH = k_cache.shape[1], k_cache.shape[2]
    out = np.empty((B, H, HD), dtype=np.uint16)
    f32 = np.empty((B, H, HD), dtype=np.float32) if return_f32 else None
    load().hkv_oracle_decode(as_u16(q), as_u16(k_cache), as_u16(v_cache), out,
                             f32.ctypes.data if f32 is not None else None, B,
                             np.ascontiguousarray(total, dtype=np.int32), H, KVH, HD, slots, 0,
                             float(scale), window, layout, mode, threads)
    return (out.view(np.float16), f32) if return_f32 else out.view(np.float16)


def prefill(q, k_cache, v_cache, past_len, scale, window=0, q_begin=0, q_end=None, threads=1):
    """q [S_new, H, HD]; planes [slots, KVH, HD] (batch 1)."""
    S_new, H, HD = q.shape
    slots, KVH = k_cache.shape[-3], k_cache.shape[-2]
    out = np.zeros((S_new, H, HD), dtype=np.uint16)
    load().hkv_oracle_prefill(as_u16(q), as_u16(k_cache), as_u16(v_cache), out, None, S_new, past_len,
                              H, KVH, HD, slots, float(scale), window, q_begin,
                              S_new if q_end is None else q_end, threads)
    return out.view(np.float16)


def qk_norm_rope(q, k, v, q_w, k_w, pos, k_cache=None, v_cache=None, rotary_dim=0, layout=0, eps=1e-6,
                 theta=10000.0, scaling=1.0):
    """In place: q [B,S,H,HD] normalised + rotated; k [B,S,KVH,HD] either rewritten in place
    (no cache) or written, with v, into k_cache / v_cache [B, slots, KVH, HD] at pos[b] + s."""
    B, S, H, HD = q.shape
    KVH = k.shape[2]
    qv, kv = as_u16(q), as_u16(k)
    assert np.shares_memory(qv, q) and np.shares_memory(kv, k)
    slots = k_cache.shape[1] if k_cache is not None else 0
    kc = as_u16(k_cache).ctypes.data if k_cache is not None else None
    vc = as_u16(v_cache).ctypes.data if v_cache is not None else None
    vv = as_u16(v).ctypes.data if v is not None else None
    load().hkv_oracle_qk_norm_rope(qv, kv, vv, as_u16(q_w), as_u16(k_w), kc, vc, B, S, H, KVH, HD, rotary_dim,
                                   np.ascontiguousarray(pos, dtype=np.int32), slots, layout, eps, theta, scaling)


def gemma4_layout(head_dim, is_global, shared, kvh, batch, max_seq, ring_window=0):
    n = len(head_dim)
    source = np.zeros(n, dtype=np.int32)
    offset = np.zeros(n, dtype=np.int64)
    rows = np.zeros(n, dtype=np.int32)
    total = load().hkv_oracle_gemma4_layout(n, shared, np.asarray(head_dim, dtype=np.int32),
                                            np.asarray(is_global, dtype=np.int32), kvh, batch, max_seq,
                                            ring_window, source, offset, rows)
    return total, source, offset, rows


def within_tolerance(x, ref, atol=2e-3, rtol=1e-2):
    """The path's acceptance rule for fp16 attention outputs: |x - ref| <= 2e-3 + 1e-2*|ref|."""
    x = np.asarray(x, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    err = np.abs(x - ref)
    ok = err <= atol + rtol * np.abs(ref)
    return bool(ok.all()), float(err.max(initial=0.0))


# ---------------------------------------------------------------------------
# The reference's own kernels (GPU only), through oracle/ref_shim.cu
# ---------------------------------------------------------------------------
_ref = None


def load_reference():
    """Returns the ctypes handle of oracle/_ref/libhector_ref_attention.so or None."""
    global _ref
    if _ref is not None:
        return _ref
    if not os.path.exists(REF_LIB):
        return None
    lib = C.CDLL(REF_LIB)
    vp = C.c_void_p
    lib.hector_ref_kv_cache_update.argtypes = [vp, vp, vp, vp] + [C.c_int] * 6 + [vp]
    lib.hector_ref_kv_cache_update_dp.argtypes = [vp, vp, vp, vp] + [C.c_int] * 5 + [vp, vp]
    lib.hector_ref_attention_cached.argtypes = [vp, vp, vp, vp] + [C.c_int] * 6 + [C.c_float, C.c_int, vp]
    lib.hector_ref_attention_cached_dp.argtypes = [vp, vp, vp, vp, C.c_int, vp] + [C.c_int] * 4 + [C.c_float, C.c_int, vp]
    lib.hector_ref_attention_prefill_cached.argtypes = [vp, vp, vp, vp] + [C.c_int] * 6 + [C.c_float, C.c_int, vp]
    if hasattr(lib, "hector_ref_qk_norm_rope_kv"):
        lib.hector_ref_qk_norm_rope.argtypes = [vp, vp, vp, vp] + [C.c_int] * 7 + [C.c_float] * 3 + [vp]
        lib.hector_ref_qk_norm_rope_kv.argtypes = ([vp] * 7 + [C.c_int] * 7 + [vp, C.c_int] + [C.c_float] * 3 + [vp])
    _ref = lib
    return lib
