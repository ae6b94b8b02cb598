// hkv_kv_cache.hpp — C++ owner of the K/V planes with the reference's layout and position
// bookkeeping (reference src/kv_cache.hpp:27-124, :161-249), extended with a per-sequence
// device position array and optional ring planes for sliding-window layers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

namespace hkv {

struct KVCacheConfig {
    uint32_t num_layers = 0;
    uint32_t num_kv_heads = 0;
    uint32_t head_dim = 0;
    uint32_t max_batch_size = 1;
    uint32_t max_seq_len = 2048;  // rows per sequence ("slots"); a ring layer uses its window
    size_t bytes_per_layer() const {
        return 2ull * max_batch_size * max_seq_len * num_kv_heads * head_dim * sizeof(half);
    }
    size_t total_bytes() const { return num_layers * bytes_per_layer(); }
};

class KVCache {
public:
    KVCache() = default;
    ~KVCache() { free(); }
    KVCache(const KVCache&) = delete;
    KVCache& operator=(const KVCache&) = delete;

    // Two planes [layers][batch][max_seq][kv_heads][head_dim] fp16, zero-filled.
    bool allocate(const KVCacheConfig& cfg) {
        if (!cfg.num_layers || !cfg.num_kv_heads || !cfg.head_dim || !cfg.max_seq_len || !cfg.max_batch_size)
            return false;
        free();
        cfg_ = cfg;
        layer_stride_ = (size_t)cfg.max_batch_size * cfg.max_seq_len * cfg.num_kv_heads * cfg.head_dim;
        const size_t bytes = cfg.num_layers * layer_stride_ * sizeof(half);
        if (cudaMalloc(&k_, bytes) != cudaSuccess) { k_ = nullptr; cudaGetLastError(); return false; }
        if (cudaMalloc(&v_, bytes) != cudaSuccess) { cudaFree(k_); k_ = v_ = nullptr; cudaGetLastError(); return false; }
        if (cudaMalloc(&d_pos_, sizeof(int32_t) * 2 * cfg.max_batch_size) != cudaSuccess) { free(); return false; }
        cudaMemset(k_, 0, bytes);
        cudaMemset(v_, 0, bytes);
        cudaMemset(d_pos_, 0, sizeof(int32_t) * 2 * cfg.max_batch_size);
        h_pos_.assign(2 * cfg.max_batch_size, 0);
        position_ = 0;
        return true;
    }
    void free() {
        if (k_) cudaFree(k_);
        if (v_) cudaFree(v_);
        if (d_pos_) cudaFree(d_pos_);
        k_ = v_ = nullptr;
        d_pos_ = nullptr;
        position_ = 0;
        layer_stride_ = 0;
    }
    bool is_allocated() const { return k_ != nullptr; }
    half* k_cache(uint32_t layer) { return (k_ && layer < cfg_.num_layers) ? k_ + layer * layer_stride_ : nullptr; }
    half* v_cache(uint32_t layer) { return (v_ && layer < cfg_.num_layers) ? v_ + layer * layer_stride_ : nullptr; }
    const KVCacheConfig& config() const { return cfg_; }

    // Host position of a batch-1 session, as in the reference.
    uint32_t position() const { return position_; }
    void advance(uint32_t n = 1) {
        position_ += n;
        if (position_ > cfg_.max_seq_len) position_ = cfg_.max_seq_len;
    }
    void rewind_to(uint32_t pos) { if (pos <= position_) position_ = pos; }
    void reset() { position_ = 0; }

    // Per-sequence device positions: d_cache_pos()[b] = write index, d_total_seq()[b] = index + 1.
    int32_t* d_cache_pos() const { return d_pos_; }
    int32_t* d_total_seq() const { return d_pos_ ? d_pos_ + cfg_.max_batch_size : nullptr; }
    // Refreshes both arrays with async copies on `stream` (outside a captured graph).
    void set_positions(const int32_t* cache_pos, cudaStream_t stream) {
        const uint32_t B = cfg_.max_batch_size;
        for (uint32_t b = 0; b < B; ++b) { h_pos_[b] = cache_pos[b]; h_pos_[B + b] = cache_pos[b] + 1; }
        cudaMemcpyAsync(d_pos_, h_pos_.data(), sizeof(int32_t) * 2 * B, cudaMemcpyHostToDevice, stream);
    }

private:
    KVCacheConfig cfg_;
    half* k_ = nullptr;
    half* v_ = nullptr;
    int32_t* d_pos_ = nullptr;
    std::vector<int32_t> h_pos_;
    uint32_t position_ = 0;
    size_t layer_stride_ = 0;
};

}  // namespace hkv
