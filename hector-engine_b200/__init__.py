"""hkv — B200-native KV-cache append + cached grouped-query attention (one hot path of
the Héctor / HELIOS engine) behind a C ABI. This package is the host-side harness around
libhkv.so: a ctypes binding, operator wrappers named like the reference's launchers and
cache owners mirroring the reference's cache objects. It has no CPU compute path."""
from . import _capi
from ._capi import (FLAG_APPEND_ONLY, FLAG_SCALAR_POSITION, HkvError, HkvGeometry, KERNEL_AUTO,
                    KERNEL_GENERIC, KERNEL_TMA, LAYOUT_LINEAR, LAYOUT_RING)
from .cache import (Gemma4KVCache, Gemma4Layer, Gemma4Layout, KVCache, KVCacheConfig,
                    gemma4_layout)
from . import dist, ops
from .ops import (Context, Geometry, clear_context_cache, decode_attention_static, fill_synthetic,
                  launch_attention_cached_fp16, launch_attention_cached_fp16_dp,
                  launch_attention_prefill_cached_fp16, launch_kv_cache_update,
                  launch_kv_cache_update_dp)

__all__ = [n for n in dir() if not n.startswith("_")]
