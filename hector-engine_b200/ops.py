"""Host-side operator interface over libhkv, mirroring the reference's launcher level
(kernels/kernels.hpp:414-483 of the reference): same names, argument meaning and error
behaviour, with tensors given as torch CUDA tensors (or raw device addresses).

PyTorch is used only for device memory and streams; all compute is in libhkv's kernels.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

from . import _capi
from ._capi import HkvError, HkvGeometry


def _ptr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    return x.data_ptr()


def _stream(stream) -> int:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


@dataclass
class Geometry:
    """Python view of `hkv_geometry`. `slots` is the reference's max_seq_len."""
    batch: int = 1
    num_heads: int = 32          # reference default (kernels/register_kernels.cpp:851)
    num_kv_heads: int | None = None  # default = num_heads (:852)
    head_dim: int = 128          # (:853)
    slots: int = 2048            # (:856)
    window_size: int = 0         # (:857)
    layout: int = _capi.LAYOUT_LINEAR
    chunk_tiles: int = 0
    batch_stride_elems: int = 0
    shard_rank: int = 0
    shard_count: int = 1
    shard_block: int = 1024
    kernel_select: int = _capi.KERNEL_AUTO
    max_seq_new: int = 0
    flags: int = 0                 # FLAG_SCALAR_POSITION | FLAG_APPEND_ONLY
    tune_prefill_splits: int = 0   # 0 = the library's own choice (parity tests force each variant)
    tune_prefill_kernel: int = 0
    tune_tma_groups: int = 0
    q_seq_stride_elems: int = 0       # decode calls: q / k_new / v_new as views into a fused QKV activation
    new_kv_seq_stride_elems: int = 0

    def to_c(self) -> HkvGeometry:
        g = HkvGeometry()
        g.batch, g.num_heads = self.batch, self.num_heads
        g.num_kv_heads = self.num_heads if self.num_kv_heads is None else self.num_kv_heads
        g.head_dim, g.slots, g.window_size = self.head_dim, self.slots, self.window_size
        g.layout, g.chunk_tiles = self.layout, self.chunk_tiles
        g.batch_stride_elems = self.batch_stride_elems
        g.shard_rank, g.shard_count, g.shard_block = self.shard_rank, self.shard_count, self.shard_block
        g.kernel_select, g.max_seq_new, g.flags = self.kernel_select, self.max_seq_new, self.flags
        g.tune_prefill_splits, g.tune_prefill_kernel = self.tune_prefill_splits, self.tune_prefill_kernel
        g.tune_tma_groups = self.tune_tma_groups
        g.q_seq_stride_elems, g.new_kv_seq_stride_elems = self.q_seq_stride_elems, self.new_kv_seq_stride_elems
        return g

    @property
    def default_scale(self) -> float:
        """1/sqrt(head_dim), the reference default (src/command.cpp:160)."""
        return 1.0 / math.sqrt(float(self.head_dim))


class Context:
    """Owns one `hkv_ctx` (split-K workspace + status word) for one layer geometry."""

    def __init__(self, geometry: Geometry):
        self.lib = _capi.load()
        self.geometry = geometry
        self._g = geometry.to_c()
        handle = C.c_void_p()
        st = self.lib.hkv_ctx_create(C.byref(handle), C.byref(self._g))
        self._h = handle
        if st != _capi.HKV_OK:
            msg = self.lib.hkv_ctx_last_error(handle).decode() if handle else "allocation failed"
            self.close()
            raise HkvError(st, msg)

    # -- lifetime -------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self.lib.hkv_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st: int):
        if st != _capi.HKV_OK:
            raise HkvError(st, self.lib.hkv_ctx_last_error(self._h).decode())

    @property
    def kernel(self) -> int:
        return self.lib.hkv_ctx_kernel(self._h)

    @property
    def launches_per_decode(self) -> int:
        return self.lib.hkv_ctx_launches_per_decode(self._h)

    @property
    def workspace_bytes(self) -> int:
        return self.lib.hkv_workspace_bytes(C.byref(self._g))

    def device_status(self, stream=None) -> int:
        out = C.c_int32(0)
        st = self.lib.hkv_ctx_device_status(self._h, _stream(stream), C.byref(out))
        if st not in (_capi.HKV_OK, 8):
            self._check(st)
        return out.value

    def selftest_bounded_wait(self, limit_ms: int = 50, stream=None):
        """Enqueues the bounded-wait self-test (a wait nothing satisfies); see device_status()."""
        self._check(self.lib.hkv_ctx_selftest_bounded_wait(self._h, limit_ms, _stream(stream)))

    def profile_begin(self, max_calls: int):
        self._check(self.lib.hkv_ctx_profile_begin(self._h, max_calls))

    def profile_end(self, stream=None):
        """-> (decode kernel ms summed, combine kernel ms summed, timed calls)."""
        d, m, n = C.c_float(0), C.c_float(0), C.c_int32(0)
        self._check(self.lib.hkv_ctx_profile_end(self._h, _stream(stream), C.byref(d), C.byref(m),
                                                 C.byref(n)))
        return d.value, m.value, n.value

    # -- the path -------------------------------------------------------------
    def append(self, k_new, v_new, k_cache, v_cache, d_cache_pos, seq_new=1, stream=None):
        self._check(self.lib.hkv_append(self._h, _ptr(k_new), _ptr(v_new), _ptr(k_cache),
                                        _ptr(v_cache), _ptr(d_cache_pos), seq_new, _stream(stream)))

    def append_at(self, k_new, v_new, k_cache, v_cache, position, seq_new=1, stream=None):
        self._check(self.lib.hkv_append_at(self._h, _ptr(k_new), _ptr(v_new), _ptr(k_cache),
                                           _ptr(v_cache), position, seq_new, _stream(stream)))

    def decode_attention(self, q, k_cache, v_cache, out, d_total_seq, scale=None, stream=None):
        scale = self.geometry.default_scale if scale is None else scale
        self._check(self.lib.hkv_decode_attention(self._h, _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                                  _ptr(out), _ptr(d_total_seq), scale, _stream(stream)))

    def decode_attention_len(self, q, k_cache, v_cache, out, seq_len, scale=None, stream=None):
        scale = self.geometry.default_scale if scale is None else scale
        self._check(self.lib.hkv_decode_attention_len(self._h, _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                                      _ptr(out), seq_len, scale, _stream(stream)))

    def append_decode_attention(self, q, k_new, v_new, k_cache, v_cache, out, d_cache_pos,
                                scale=None, stream=None):
        scale = self.geometry.default_scale if scale is None else scale
        self._check(self.lib.hkv_append_decode_attention(
            self._h, _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), _ptr(out),
            _ptr(d_cache_pos), scale, _stream(stream)))

    def append_decode_attention_host(self, h_q, h_k_new, h_v_new, k_cache, v_cache, h_out,
                                     d_cache_pos, scale=None, stream=None):
        scale = self.geometry.default_scale if scale is None else scale
        self._check(self.lib.hkv_append_decode_attention_host(
            self._h, _ptr(h_q), _ptr(h_k_new), _ptr(h_v_new), _ptr(k_cache), _ptr(v_cache),
            _ptr(h_out), _ptr(d_cache_pos), scale, _stream(stream)))

    def append_decode_attention_host_pipelined(self, h_q, h_k_new, h_v_new, k_cache, v_cache, h_out,
                                               d_cache_pos, scale=None, stream=None):
        """As append_decode_attention_host, with the copies on the context's own streams so that they
        overlap neighbouring calls' kernels; h_out is complete after host_flush() + a sync of `stream`."""
        scale = self.geometry.default_scale if scale is None else scale
        self._check(self.lib.hkv_append_decode_attention_host_pipelined(
            self._h, _ptr(h_q), _ptr(h_k_new), _ptr(h_v_new), _ptr(k_cache), _ptr(v_cache),
            _ptr(h_out), _ptr(d_cache_pos), scale, _stream(stream)))

    def host_flush(self, stream=None):
        self._check(self.lib.hkv_host_flush(self._h, _stream(stream)))

    def prefill_attention(self, q, k_cache, v_cache, out, seq_new, past_len, scale=None, stream=None):
        scale = self.geometry.default_scale if scale is None else scale
        self._check(self.lib.hkv_prefill_attention(self._h, _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                                   _ptr(out), seq_new, past_len, scale, _stream(stream)))

    def prefill_append_attention(self, q, k_new, v_new, k_cache, v_cache, out, seq_new, past_len, scale=None, stream=None):
        """Append a chunk's K/V rows at past_len and attend its queries over the cache — for a ring plane
        of exactly `window` rows in the order attend, then append (hkv_prefill_append_attention)."""
        scale = self.geometry.default_scale if scale is None else scale
        self._check(self.lib.hkv_prefill_append_attention(self._h, _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(k_cache),
                                                          _ptr(v_cache), _ptr(out), seq_new, past_len, scale,
                                                          _stream(stream)))

    def plan_prefill(self, seq_new: int, past_len: int, sm_count: int | None = None):
        """Host plan of one prefill_attention call -> (query tiles in flight per CTA: 2, 1, or 0 for the
        SIMT kernel; work items; key-range splits; shortest key span in tiles)."""
        if sm_count is None:
            import torch
            sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        vals = [C.c_int32() for _ in range(4)]
        self._check(self.lib.hkv_plan_prefill(C.byref(self._g), seq_new, past_len, sm_count, *[C.byref(v) for v in vals]))
        return tuple(v.value for v in vals)

    def qk_norm_rope_kv(self, q, k, v, q_norm_w, k_norm_w, k_cache=None, v_cache=None, d_cache_pos=None,
                        position=0, seq_new=1, rotary_dim=0, eps=1e-6, theta=10000.0, scaling_factor=1.0,
                        stream=None):
        """Per-head RMSNorm(q, k) + RoPE, K/V written into the cache when planes are given
        (reference launch_qk_norm_rope_kv_fp16, kernels/attention.cu:947-973)."""
        self._check(self.lib.hkv_qk_norm_rope_kv(
            self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(k_cache), _ptr(v_cache),
            _ptr(d_cache_pos), position, seq_new, rotary_dim, eps, theta, scaling_factor, _stream(stream)))

    def decode_partials(self, q, k_new, v_new, k_cache, v_cache, partial_out, d_total_seq,
                        scale=None, stream=None):
        scale = self.geometry.default_scale if scale is None else scale
        self._check(self.lib.hkv_decode_partials(
            self._h, _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache),
            _ptr(partial_out), _ptr(d_total_seq), scale, _stream(stream)))

    def combine_partials(self, partials, num_parts, out, stream=None):
        self._check(self.lib.hkv_combine_partials(self._h, _ptr(partials), num_parts, _ptr(out),
                                                  _stream(stream)))

    # -- peer exchange (peer-mapped mailboxes instead of a collective) ----------------
    def exchange_bytes(self, world: int) -> int:
        n = C.c_size_t(0)
        self._check(self.lib.hkv_exchange_bytes(self._h, world, C.byref(n)))
        return int(n.value)

    @staticmethod
    def make_exchange(rank: int, mailboxes, wait_limit_ms: int = 0):
        """`mailboxes[r]`: rank r's mailbox as this process addresses it (a zeroed uint8 tensor of
        exchange_bytes(world) bytes, or a raw pointer for a peer's mapped allocation)."""
        x = _capi.HkvExchange()
        x.rank, x.world, x.wait_limit_ms = rank, len(mailboxes), wait_limit_ms
        for r, m in enumerate(mailboxes):
            x.mailbox[r] = m if isinstance(m, int) else _ptr(m)
        return x

    def decode_partials_publish(self, q, k_new, v_new, k_cache, v_cache, exchange, d_total_seq, scale=None,
                             stream=None):
        scale = self.geometry.default_scale if scale is None else scale
        self._check(self.lib.hkv_decode_partials_publish(
            self._h, _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), C.byref(exchange),
            _ptr(d_total_seq), scale, _stream(stream)))

    def merge_published(self, exchange, out, stream=None):
        self._check(self.lib.hkv_merge_published(self._h, C.byref(exchange), _ptr(out), _stream(stream)))


STATIC_SCRATCH_BYTES = 8 << 20


def decode_attention_static(geometry: Geometry, q, k_cache, v_cache, out, d_total_seq, scale=None,
                            stream=None):
    """Decode attention without a Context and without any allocation: the split-K partials
    use the library's fixed 8 MiB array (hkv_decode_attention_static). For callers that may
    not allocate device memory when they need attention; calls must not overlap on the GPU."""
    lib = _capi.load()
    scale = geometry.default_scale if scale is None else scale
    g = geometry.to_c()
    st = lib.hkv_decode_attention_static(C.byref(g), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out),
                                         _ptr(d_total_seq), scale, _stream(stream))
    if st != _capi.HKV_OK:
        raise HkvError(st, lib.hkv_status_string(st).decode())


def fill_synthetic(dst, seed: int, first_index: int = 0, count: int | None = None, stream=None):
    """Fills an fp16 CUDA tensor with the deterministic synthetic stream (see hkv_fill_synthetic)."""
    lib = _capi.load()
    n = dst.numel() if count is None else count
    st = lib.hkv_fill_synthetic(_ptr(dst), seed & 0xFFFFFFFFFFFFFFFF, first_index, n, _stream(stream))
    if st != _capi.HKV_OK:
        raise HkvError(st, "hkv_fill_synthetic")


# ---------------------------------------------------------------------------
# Reference-named launchers (kernels/kernels.hpp:414-483): one-shot forms that build a
# context per call signature and cache it, for tests that read like the reference's.
# They keep the reference's position convention: `d_position` / `d_seq_len` is ONE int32
# on the device that every sequence of the batch reads (kernels/attention.cu:351, :1129),
# not the per-sequence arrays of Context.append / Context.decode_attention.
# ---------------------------------------------------------------------------
_ctx_cache: dict[tuple, Context] = {}


def _ctx_for(**kw) -> Context:
    key = tuple(sorted(kw.items()))
    ctx = _ctx_cache.get(key)
    if ctx is None:
        ctx = _ctx_cache[key] = Context(Geometry(**kw))
    return ctx


def launch_kv_cache_update(new_k, new_v, k_cache, v_cache, batch_size, seq_len, kv_heads, head_dim,
                           max_seq_len, position, stream=None, **geom):
    ctx = _ctx_for(batch=batch_size, num_heads=kv_heads, num_kv_heads=kv_heads, head_dim=head_dim,
                   slots=max_seq_len, flags=_capi.FLAG_APPEND_ONLY, **geom)
    ctx.append_at(new_k, new_v, k_cache, v_cache, position, seq_len, stream)


def launch_kv_cache_update_dp(new_k, new_v, k_cache, v_cache, batch_size, seq_len, kv_heads,
                              head_dim, max_seq_len, d_position, stream=None, **geom):
    ctx = _ctx_for(batch=batch_size, num_heads=kv_heads, num_kv_heads=kv_heads, head_dim=head_dim,
                   slots=max_seq_len, flags=_capi.FLAG_APPEND_ONLY | _capi.FLAG_SCALAR_POSITION, **geom)
    ctx.append(new_k, new_v, k_cache, v_cache, d_position, seq_len, stream)


def launch_attention_cached_fp16(q, k_cache, v_cache, output, batch_size, seq_len, num_heads,
                                 num_kv_heads, head_dim, max_seq_len, scale, window_size,
                                 stream=None, **geom):
    ctx = _ctx_for(batch=batch_size, num_heads=num_heads, num_kv_heads=num_kv_heads,
                   head_dim=head_dim, slots=max_seq_len, window_size=window_size, **geom)
    ctx.decode_attention_len(q, k_cache, v_cache, output, seq_len, scale, stream)


def launch_attention_cached_fp16_dp(q, k_cache, v_cache, output, batch_size, d_seq_len, num_heads,
                                    num_kv_heads, head_dim, max_seq_len, scale, window_size,
                                    stream=None, **geom):
    ctx = _ctx_for(batch=batch_size, num_heads=num_heads, num_kv_heads=num_kv_heads,
                   head_dim=head_dim, slots=max_seq_len, window_size=window_size,
                   flags=_capi.FLAG_SCALAR_POSITION, **geom)
    ctx.decode_attention(q, k_cache, v_cache, output, d_seq_len, scale, stream)


def launch_attention_prefill_cached_fp16(q, k_cache, v_cache, output, seq_new, past_len, num_heads,
                                         num_kv_heads, head_dim, max_seq_len, scale, window_size,
                                         stream=None, **geom):
    # key-split workspace rounded to 512..4096 queries (as the C++ adapter does): ragged chunk
    # lengths share a context; longer chunks have enough work items without a split
    cap = next((c for c in (512, 1024, 2048, 4096) if seq_new <= c), 0)
    ctx = _ctx_for(batch=1, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                   slots=max_seq_len, window_size=window_size, max_seq_new=cap, **geom)
    ctx.prefill_attention(q, k_cache, v_cache, output, seq_new, past_len, scale, stream)


def clear_context_cache():
    for ctx in _ctx_cache.values():
        ctx.close()
    _ctx_cache.clear()
