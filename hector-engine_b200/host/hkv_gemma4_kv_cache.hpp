// hkv_gemma4_kv_cache.hpp — C++ owner of a heterogeneous / shared KV cache, the layout of the
// reference's Gemma4KVCache (reference src/gemma4_kv_cache.hpp:39-114, :132-145, :147-187):
//   * the first (layers - num_kv_shared_layers) layers own physical slots, laid out back to back
//     in one K plane and one V plane, each slot [batch][rows][kv_heads][head_dim of THAT layer];
//   * later local layers alias the last local owner, later global layers the last global owner
//     (true pointer aliases; the head_dim must match the owner's);
//   * planes are zero-filled; tensors are published as `<prefix>.layerN.k` / `.v` with shape
//     {batch, rows, kv_heads, head_dim(N)}; host position bookkeeping as KVCache.
// One extension: with `ring_window` > 0 the local (sliding-window) owners get ring planes of
// `ring_window` rows indexed position mod ring_window instead of max_seq_len rows. The ring must hold
// the layers' sliding window; attention over it equals the reference's linear plane with the same
// window. Exactly the window is the smallest plane; window + prefill chunk - 1 rows (a multiple of 64)
// lets a chunked prefill append before it attends, and costs decode nothing (the decode kernel reads
// only the tiles the window touches).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <limits>
#include <stdexcept>
#include <string>
#include <vector>

namespace hkv {

// What the layout needs to know of a layer (the reference reads the same three facts from its
// per-layer model config: head_dim, is_global_attention(), sliding_window).
struct Gemma4LayerSpec {
    uint32_t head_dim = 0;
    bool is_global = false;
    uint32_t sliding_window = 0;   // 0 for global layers
};

class Gemma4KVCache {
public:
    Gemma4KVCache() = default;
    ~Gemma4KVCache() { free(); }
    Gemma4KVCache(const Gemma4KVCache&) = delete;
    Gemma4KVCache& operator=(const Gemma4KVCache&) = delete;

    // Returns false (and leaves the object empty) exactly where the reference's allocate() does:
    // no layers, a zero dimension, more shared layers than layers, no owner at all, a shared layer
    // without an owner of its kind or with another head_dim, size overflow, or a failed allocation.
    bool allocate(const std::vector<Gemma4LayerSpec>& layers, uint32_t num_kv_shared_layers, uint32_t num_kv_heads,
                  uint32_t max_batch_size, uint32_t max_seq_len, uint32_t ring_window = 0) {
        free();
        if (layers.empty() || num_kv_heads == 0 || max_batch_size == 0 || max_seq_len == 0 ||
            num_kv_shared_layers > layers.size())
            return false;
        const uint32_t n = (uint32_t)layers.size();
        const uint32_t first_shared = n - num_kv_shared_layers;
        if (first_shared == 0) return false;
        num_kv_heads_ = num_kv_heads;
        max_batch_size_ = max_batch_size;
        max_seq_len_ = max_seq_len;
        first_shared_layer_ = first_shared;
        specs_ = layers;
        source_.resize(n);
        offsets_.resize(n);
        rows_.resize(n);
        int32_t last_local = -1, last_global = -1;
        size_t total = 0;
        for (uint32_t i = 0; i < first_shared; ++i) {
            if (layers[i].head_dim == 0) return fail_layout();
            source_[i] = i;
            offsets_[i] = total;
            rows_[i] = (!layers[i].is_global && ring_window > 0) ? (ring_window < max_seq_len ? ring_window : max_seq_len)
                                                                  : max_seq_len;
            if (layers[i].is_global) last_global = (int32_t)i;
            else last_local = (int32_t)i;
            size_t stride = 0;
            if (!checked_stride(rows_[i], layers[i].head_dim, stride) || total > std::numeric_limits<size_t>::max() - stride)
                return fail_layout();
            total += stride;
        }
        for (uint32_t i = first_shared; i < n; ++i) {
            const int32_t src = layers[i].is_global ? last_global : last_local;
            if (src < 0 || layers[i].head_dim != layers[(size_t)src].head_dim) return fail_layout();
            source_[i] = (uint32_t)src;
            offsets_[i] = offsets_[(size_t)src];
            rows_[i] = rows_[(size_t)src];
        }
        if (total == 0 || total > std::numeric_limits<size_t>::max() / sizeof(half)) return fail_layout();
        elements_per_plane_ = total;
        const size_t bytes = total * sizeof(half);
        if (cudaMalloc(&k_data_, bytes) != cudaSuccess) { k_data_ = nullptr; cudaGetLastError(); return fail_layout(); }
        if (cudaMalloc(&v_data_, bytes) != cudaSuccess) { v_data_ = nullptr; cudaGetLastError(); return fail_layout(); }
        if (cudaMemset(k_data_, 0, bytes) != cudaSuccess || cudaMemset(v_data_, 0, bytes) != cudaSuccess) return fail_layout();
        position_ = 0;
        return true;
    }

    void free() {
        if (k_data_) cudaFree(k_data_);
        if (v_data_) cudaFree(v_data_);
        k_data_ = v_data_ = nullptr;
        specs_.clear();
        source_.clear();
        offsets_.clear();
        rows_.clear();
        num_kv_heads_ = max_batch_size_ = max_seq_len_ = first_shared_layer_ = 0;
        elements_per_plane_ = 0;
        position_ = 0;
    }

    // Publishes every layer's planes under the reference's names. `reg(name, pointer, shape)` is the
    // engine's registration of an external fp16 tensor (for the reference engine:
    // engine.tensors().register_external(name, pointer, shape, dtype::FP16())).
    template <class Register>
    void register_tensors(Register&& reg, const std::string& prefix) {
        if (!is_allocated()) throw std::runtime_error("Gemma4KVCache: cache is not allocated");
        for (uint32_t layer = 0; layer < num_layers(); ++layer) {
            const std::vector<uint32_t> shape{max_batch_size_, rows_[layer], num_kv_heads_, specs_[layer].head_dim};
            const std::string base = prefix + ".layer" + std::to_string(layer);
            reg(base + ".k", k_cache(layer), shape);
            reg(base + ".v", v_cache(layer), shape);
        }
    }

    half* k_cache(uint32_t layer) { return valid_layer(layer) ? k_data_ + offsets_[layer] : nullptr; }
    const half* k_cache(uint32_t layer) const { return valid_layer(layer) ? k_data_ + offsets_[layer] : nullptr; }
    half* v_cache(uint32_t layer) { return valid_layer(layer) ? v_data_ + offsets_[layer] : nullptr; }
    const half* v_cache(uint32_t layer) const { return valid_layer(layer) ? v_data_ + offsets_[layer] : nullptr; }

    bool is_allocated() const { return k_data_ && v_data_; }
    uint32_t num_layers() const { return (uint32_t)source_.size(); }
    uint32_t physical_slots() const { return first_shared_layer_; }
    uint32_t first_shared_layer() const { return first_shared_layer_; }
    uint32_t source_layer(uint32_t layer) const {
        return layer < source_.size() ? source_[layer] : std::numeric_limits<uint32_t>::max();
    }
    bool is_shared(uint32_t layer) const { return layer < source_.size() && source_[layer] != layer; }
    uint32_t head_dim(uint32_t layer) const { return layer < specs_.size() ? specs_[layer].head_dim : 0; }
    bool is_global(uint32_t layer) const { return layer < specs_.size() && specs_[layer].is_global; }
    uint32_t sliding_window(uint32_t layer) const { return layer < specs_.size() ? specs_[layer].sliding_window : 0; }
    // Rows per sequence of the layer's plane: max_seq_len, or the ring size for a local ring plane.
    uint32_t rows(uint32_t layer) const { return layer < rows_.size() ? rows_[layer] : 0; }
    bool is_ring(uint32_t layer) const { return layer < rows_.size() && rows_[layer] != max_seq_len_; }
    uint32_t num_kv_heads() const { return num_kv_heads_; }
    uint32_t max_batch_size() const { return max_batch_size_; }
    uint32_t max_seq_len() const { return max_seq_len_; }
    size_t total_bytes() const { return 2 * elements_per_plane_ * sizeof(half); }

    uint32_t position() const { return position_; }
    void reset() { position_ = 0; }
    void advance(uint32_t tokens = 1) {
        position_ = tokens > max_seq_len_ - position_ ? max_seq_len_ : position_ + tokens;
    }
    void rewind_to(uint32_t position) { if (position <= position_) position_ = position; }

private:
    bool checked_stride(uint32_t rows, uint32_t head_dim, size_t& stride) const {
        size_t value = max_batch_size_;
        const size_t factors[] = {rows, num_kv_heads_, head_dim};
        for (size_t f : factors) {
            if (f == 0 || value > std::numeric_limits<size_t>::max() / f) return false;
            value *= f;
        }
        stride = value;
        return true;
    }
    bool fail_layout() { free(); return false; }
    bool valid_layer(uint32_t layer) const { return is_allocated() && layer < offsets_.size(); }

    half* k_data_ = nullptr;
    half* v_data_ = nullptr;
    std::vector<Gemma4LayerSpec> specs_;
    std::vector<uint32_t> source_;
    std::vector<size_t> offsets_;
    std::vector<uint32_t> rows_;
    uint32_t num_kv_heads_ = 0, max_batch_size_ = 0, max_seq_len_ = 0, first_shared_layer_ = 0;
    size_t elements_per_plane_ = 0;
    uint32_t position_ = 0;
};

}  // namespace hkv
