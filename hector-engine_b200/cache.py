"""KV-cache owners mirroring the reference's cache objects.

  KVCacheConfig / KVCache   src/kv_cache.hpp:27-124, :161-249 of the reference
  Gemma4KVCache             src/gemma4_kv_cache.hpp:22-240 of the reference

Same layout, zero fill, position bookkeeping (advance clamps, rewind_to only moves
back) and shared-layer aliasing. Added over the reference: a per-sequence DEVICE position
array (the reference keeps one scalar, src/engine.hpp:206-207) and an optional ring
layout for sliding-window layers (`ring_window`). Device memory comes from torch; the
layout arithmetic is plain Python and runs without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class KVCacheConfig:
    num_layers: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    max_batch_size: int = 1
    max_seq_len: int = 2048

    def bytes_per_layer(self) -> int:
        return 2 * self.max_batch_size * self.max_seq_len * self.num_kv_heads * self.head_dim * 2

    def total_bytes(self) -> int:
        return self.num_layers * self.bytes_per_layer()


class _PositionMixin:
    _position: int = 0
    _max_seq: int = 0

    def position(self) -> int:
        return self._position

    def advance(self, num_tokens: int = 1) -> None:
        self._position = min(self._position + num_tokens, self._max_seq)  # clamp, never overflow

    def rewind_to(self, pos: int) -> None:
        if pos <= self._position:
            self._position = pos

    def reset(self) -> None:
        self._position = 0


class KVCache(_PositionMixin):
    """Two planes K and V, each [layers][batch][max_seq][kv_heads][head_dim] fp16, zeroed."""

    def __init__(self):
        self.config = KVCacheConfig()
        self.k_data = None
        self.v_data = None
        self.layer_stride = 0

    def allocate(self, config: KVCacheConfig, device="cuda") -> bool:
        if min(config.num_layers, config.num_kv_heads, config.head_dim, config.max_seq_len) <= 0:
            return False
        import torch
        self.free()
        self.config = config
        self._max_seq = config.max_seq_len
        self.layer_stride = (config.max_batch_size * config.max_seq_len * config.num_kv_heads *
                             config.head_dim)
        n = config.num_layers * self.layer_stride
        try:
            self.k_data = torch.zeros(n, dtype=torch.float16, device=device)
            self.v_data = torch.zeros(n, dtype=torch.float16, device=device)
        except RuntimeError:
            self.free()
            return False
        self._position = 0
        return True

    def free(self) -> None:
        self.k_data = self.v_data = None
        self.layer_stride = 0
        self._position = 0

    def is_allocated(self) -> bool:
        return self.k_data is not None

    def _plane(self, data, layer: int):
        if data is None or not 0 <= layer < self.config.num_layers:
            return None
        c = self.config
        return data[layer * self.layer_stride:(layer + 1) * self.layer_stride].view(
            c.max_batch_size, c.max_seq_len, c.num_kv_heads, c.head_dim)

    def k_cache(self, layer: int):
        return self._plane(self.k_data, layer)

    def v_cache(self, layer: int):
        return self._plane(self.v_data, layer)

    def current_seq_len(self) -> int:
        return self._position


@dataclass
class Gemma4Layer:
    head_dim: int
    is_global: bool
    sliding_window: int = 0


@dataclass
class Gemma4Layout:
    """Result of the heterogeneous/shared layout computation (pure arithmetic)."""
    source: list = field(default_factory=list)   # owner layer of each layer's slot
    offset: list = field(default_factory=list)   # element offset into a plane
    rows: list = field(default_factory=list)     # rows per sequence (max_seq, or ring window)
    head_dim: list = field(default_factory=list)
    elements_per_plane: int = 0
    first_shared: int = 0


def gemma4_layout(layers: list, num_kv_shared_layers: int, num_kv_heads: int, max_batch_size: int,
                  max_seq_len: int, ring_window: int = 0) -> Gemma4Layout | None:
    """First (N - shared) layers own slots laid out back to back with their own head_dim;
    later local layers alias the last local owner, later global layers the last global
    owner (src/gemma4_kv_cache.hpp:39-114). Returns None where the reference's allocate()
    returns false. `ring_window` > 0 gives local owners `ring_window` rows instead of
    max_seq_len (not in the reference)."""
    n = len(layers)
    if n == 0 or num_kv_heads <= 0 or max_batch_size <= 0 or max_seq_len <= 0 or num_kv_shared_layers > n:
        return None
    first_shared = n - num_kv_shared_layers
    if first_shared == 0:
        return None
    out = Gemma4Layout(first_shared=first_shared)
    last_local = last_global = -1
    total = 0
    for i in range(first_shared):
        ly = layers[i]
        if ly.head_dim <= 0:
            return None
        rows = min(ring_window, max_seq_len) if (ring_window > 0 and not ly.is_global) else max_seq_len
        out.source.append(i)
        out.offset.append(total)
        out.rows.append(rows)
        out.head_dim.append(ly.head_dim)
        if ly.is_global:
            last_global = i
        else:
            last_local = i
        total += max_batch_size * rows * num_kv_heads * ly.head_dim
    for i in range(first_shared, n):
        ly = layers[i]
        src = last_global if ly.is_global else last_local
        if src < 0 or ly.head_dim != layers[src].head_dim:
            return None
        out.source.append(src)
        out.offset.append(out.offset[src])
        out.rows.append(out.rows[src])
        out.head_dim.append(ly.head_dim)
    if total == 0:
        return None
    out.elements_per_plane = total
    return out


class Gemma4KVCache(_PositionMixin):
    """Heterogeneous per-layer head_dim, shared-KV aliasing, optional ring planes."""

    def __init__(self):
        self.layout: Gemma4Layout | None = None
        self.k_data = self.v_data = None
        self.num_kv_heads = self.max_batch_size = 0

    def allocate(self, layers: list, num_kv_shared_layers: int, num_kv_heads: int,
                 max_batch_size: int, max_seq_len: int, ring_window: int = 0, device="cuda") -> bool:
        self.free()
        lay = gemma4_layout(layers, num_kv_shared_layers, num_kv_heads, max_batch_size, max_seq_len,
                            ring_window)
        if lay is None:
            return False
        import torch
        try:
            self.k_data = torch.zeros(lay.elements_per_plane, dtype=torch.float16, device=device)
            self.v_data = torch.zeros(lay.elements_per_plane, dtype=torch.float16, device=device)
        except RuntimeError:
            self.free()
            return False
        self.layout = lay
        self.num_kv_heads, self.max_batch_size, self._max_seq = num_kv_heads, max_batch_size, max_seq_len
        self._position = 0
        return True

    def free(self) -> None:
        self.layout = None
        self.k_data = self.v_data = None
        self._position = 0

    def is_allocated(self) -> bool:
        return self.k_data is not None

    def num_layers(self) -> int:
        return len(self.layout.source) if self.layout else 0

    def physical_slots(self) -> int:
        return self.layout.first_shared if self.layout else 0

    def source_layer(self, layer: int) -> int:
        return self.layout.source[layer] if self.layout and 0 <= layer < self.num_layers() else 0xFFFFFFFF

    def is_shared(self, layer: int) -> bool:
        return bool(self.layout) and 0 <= layer < self.num_layers() and self.layout.source[layer] != layer

    def head_dim(self, layer: int) -> int:
        return self.layout.head_dim[layer] if self.layout and 0 <= layer < self.num_layers() else 0

    def rows(self, layer: int) -> int:
        return self.layout.rows[layer] if self.layout and 0 <= layer < self.num_layers() else 0

    def total_bytes(self) -> int:
        return 2 * self.layout.elements_per_plane * 2 if self.layout else 0

    def _plane(self, data, layer: int):
        if data is None or not 0 <= layer < self.num_layers():
            return None
        lay = self.layout
        n = self.max_batch_size * lay.rows[layer] * self.num_kv_heads * lay.head_dim[layer]
        return data[lay.offset[layer]:lay.offset[layer] + n].view(
            self.max_batch_size, lay.rows[layer], self.num_kv_heads, lay.head_dim[layer])

    def k_cache(self, layer: int):
        return self._plane(self.k_data, layer)

    def v_cache(self, layer: int):
        return self._plane(self.v_data, layer)

    def tensor_names(self, prefix: str) -> dict:
        """`<prefix>.layerN.k/.v` -> (plane, shape), the names register_tensors() publishes
        (src/gemma4_kv_cache.hpp:132-145)."""
        out = {}
        for i in range(self.num_layers()):
            shape = (self.max_batch_size, self.layout.rows[i], self.num_kv_heads, self.layout.head_dim[i])
            out[f"{prefix}.layer{i}.k"] = (self.k_cache(i), shape)
            out[f"{prefix}.layer{i}.v"] = (self.v_cache(i), shape)
        return out
