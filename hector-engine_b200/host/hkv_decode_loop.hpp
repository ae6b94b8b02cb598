// hkv_decode_loop.hpp — batched decode driver for the attention path: many sessions share one
// captured CUDA graph, each in its own batch slot, and only the device position arrays change
// from token to token.
//
// What it stands in for (reference project paths):
//   * InferenceSession::Impl::forward_one (src/inference_session.cpp:248-276): per token, publish
//     the cache position to the device, run the first token un-captured, replay the captured graph
//     afterwards, advance the host position;
//   * Engine::update_device_cache_pos / execute_graph_replay (src/engine.cpp:138-187, :206-260):
//     two async 4-byte copies per token and a capture-once graph with a per-token fallback when
//     capture fails (sticky error cleared);
//   * the model-wide mutex that serialises sessions (src/inference_session.cpp:509): here sessions
//     do not take turns, they occupy slots of one batch and advance together.
//
// Three pieces, usable separately:
//   SessionBoard  — slot table + pinned, double-buffered staging of the int32[batch] position arrays;
//   GraphReplay   — capture-once replay of an enqueue callback with the engine's fallback rules;
//   BatchedDecodeLoop — an hkv_ctx per distinct layer geometry and both of the above; step()
//                   enqueues fused append + attention for every layer (with a caller hook between
//                   layers for the model's other ops) and replays it. Layers may all be alike (the
//                   loop then owns the planes) or differ per layer — head_dim, sliding window over a
//                   linear or ring plane, scale, shared layers that attend an owner's plane without
//                   appending — as in the reference's Gemma-4 graph.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <functional>
#include <map>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include "hkv.h"
#include "hkv_gemma4_kv_cache.hpp"
#include "hkv_kv_cache.hpp"

namespace hkv {

// ---------------------------------------------------------------------------
// Slot table. A free slot publishes cache_pos = -1 / total_seq = 0: the kernels then append
// nothing for it, attend nothing and write a zero output row, so the launch shape never changes.
// ---------------------------------------------------------------------------
class SessionBoard {
public:
    SessionBoard(uint32_t slots, uint32_t max_seq_len) : slots_(slots), max_seq_(max_seq_len), pos_(slots, -1) {
        if (!slots) throw std::runtime_error("SessionBoard: zero slots");
        if (cudaMalloc(&d_pos_, sizeof(int32_t) * 2 * slots) != cudaSuccess) fail("cudaMalloc");
        if (cudaMallocHost(&h_stage_, sizeof(int32_t) * 4 * slots) != cudaSuccess) fail("cudaMallocHost");
        for (int i = 0; i < 2; ++i)
            if (cudaEventCreateWithFlags(&copied_[i], cudaEventDisableTiming) != cudaSuccess) fail("cudaEventCreate");
        for (uint32_t b = 0; b < slots; ++b) { h_stage_[b] = -1; h_stage_[slots + b] = 0; }
        if (cudaMemcpy(d_pos_, h_stage_, sizeof(int32_t) * 2 * slots, cudaMemcpyHostToDevice) != cudaSuccess) fail("cudaMemcpy");
    }
    ~SessionBoard() {
        for (auto& e : copied_) if (e) cudaEventDestroy(e);
        if (h_stage_) cudaFreeHost(h_stage_);
        if (d_pos_) cudaFree(d_pos_);
    }
    SessionBoard(const SessionBoard&) = delete;
    SessionBoard& operator=(const SessionBoard&) = delete;

    uint32_t slots() const { return slots_; }
    uint32_t active_count() const { uint32_t n = 0; for (int32_t p : pos_) n += p >= 0; return n; }
    bool active(int slot) const { return slot >= 0 && (uint32_t)slot < slots_ && pos_[(size_t)slot] >= 0; }
    // Position = number of rows the session has in the cache = index of the next row.
    uint32_t position(int slot) const { return active(slot) ? (uint32_t)pos_[(size_t)slot] : 0; }

    // Takes the lowest free slot; -1 when the batch is full.
    int attach(uint32_t start_pos = 0) {
        for (uint32_t b = 0; b < slots_; ++b)
            if (pos_[b] < 0) { pos_[b] = (int32_t)(start_pos < max_seq_ ? start_pos : max_seq_); return (int)b; }
        return -1;
    }
    void detach(int slot) { if (active(slot)) pos_[(size_t)slot] = -1; }
    // Same clamping as the reference's KVCache::advance / rewind_to (src/kv_cache.hpp:100-113).
    void advance(int slot, uint32_t n = 1) {
        if (!active(slot)) return;
        const uint64_t p = (uint64_t)pos_[(size_t)slot] + n;
        pos_[(size_t)slot] = (int32_t)(p < max_seq_ ? p : max_seq_);
    }
    void advance_all(uint32_t n = 1) { for (uint32_t b = 0; b < slots_; ++b) advance((int)b, n); }
    void rewind_to(int slot, uint32_t pos) { if (active(slot) && pos <= (uint32_t)pos_[(size_t)slot]) pos_[(size_t)slot] = (int32_t)pos; }

    // Fixed device addresses, as Engine::device_cache_pos() / device_total_seq().
    int32_t* d_cache_pos() const { return d_pos_; }
    int32_t* d_total_seq() const { return d_pos_ + slots_; }

    // One async copy of both arrays on `stream` (outside any captured graph). The pinned staging
    // area is double-buffered and guarded by an event, so publishing token t+1 never rewrites the
    // buffer token t's copy may still be reading.
    void publish(cudaStream_t stream, uint32_t seq_len = 1) {
        const int buf = turn_ & 1;
        ++turn_;
        if (used_[buf] && cudaEventSynchronize(copied_[buf]) != cudaSuccess) fail("cudaEventSynchronize");
        int32_t* h = h_stage_ + (size_t)buf * 2 * slots_;
        for (uint32_t b = 0; b < slots_; ++b) {
            h[b] = pos_[b];
            h[slots_ + b] = pos_[b] >= 0 ? pos_[b] + (int32_t)seq_len : 0;
        }
        if (cudaMemcpyAsync(d_pos_, h, sizeof(int32_t) * 2 * slots_, cudaMemcpyHostToDevice, stream) != cudaSuccess)
            fail("cudaMemcpyAsync");
        if (cudaEventRecord(copied_[buf], stream) != cudaSuccess) fail("cudaEventRecord");
        used_[buf] = true;
    }

private:
    [[noreturn]] static void fail(const char* what) {
        const cudaError_t e = cudaGetLastError();
        throw std::runtime_error(std::string("SessionBoard: ") + what + ": " + cudaGetErrorString(e));
    }
    uint32_t slots_, max_seq_;
    std::vector<int32_t> pos_;       // -1 = free
    int32_t* d_pos_ = nullptr;       // [2][slots]: cache_pos, total_seq
    int32_t* h_stage_ = nullptr;     // pinned, [2 buffers][2][slots]
    cudaEvent_t copied_[2] = {nullptr, nullptr};
    bool used_[2] = {false, false};
    unsigned turn_ = 0;
};

// ---------------------------------------------------------------------------
// Capture-once replay. run() replays the graph when there is one; otherwise it captures
// `enqueue(stream)` (global capture mode, as the engine does), instantiates and launches it. If
// capture or instantiation fails the sticky error is cleared, the work is enqueued directly and
// run() returns false; the next call tries again unless `give_up_after` failures were seen.
// ---------------------------------------------------------------------------
class GraphReplay {
public:
    explicit GraphReplay(int give_up_after = 3) : give_up_after_(give_up_after) {}
    ~GraphReplay() { invalidate(); }
    GraphReplay(const GraphReplay&) = delete;
    GraphReplay& operator=(const GraphReplay&) = delete;

    bool valid() const { return exec_ != nullptr; }
    uint64_t replays() const { return replays_; }
    int capture_failures() const { return failures_; }
    const std::string& last_error() const { return last_error_; }
    size_t node_count() const { return nodes_; }

    // Drops the graph (geometry, pointers or the set of layers changed): the next run() captures again.
    void invalidate() {
        if (exec_) cudaGraphExecDestroy(exec_);
        if (graph_) cudaGraphDestroy(graph_);
        exec_ = nullptr;
        graph_ = nullptr;
        nodes_ = 0;
    }

    template <class Enqueue>
    bool run(cudaStream_t stream, Enqueue&& enqueue) {
        if (!exec_ && failures_ < give_up_after_) capture(stream, enqueue);
        if (exec_) {
            const cudaError_t e = cudaGraphLaunch(exec_, stream);
            if (e != cudaSuccess) throw std::runtime_error(std::string("GraphReplay: launch: ") + cudaGetErrorString(e));
            ++replays_;
            return true;
        }
        enqueue(stream);
        return false;
    }

private:
    template <class Enqueue>
    void capture(cudaStream_t stream, Enqueue& enqueue) {
        cudaGetLastError();
        if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeGlobal) != cudaSuccess) {
            note_failure("begin capture");
            return;
        }
        bool threw = false;
        try {
            enqueue(stream);
        } catch (const std::exception& ex) {
            threw = true;
            last_error_ = ex.what();
        }
        cudaGraph_t g = nullptr;
        const cudaError_t end = cudaStreamEndCapture(stream, &g);
        if (threw || end != cudaSuccess || !g) {
            if (g) cudaGraphDestroy(g);
            if (!threw) last_error_ = cudaGetErrorString(end);
            note_failure(nullptr);
            return;
        }
        cudaGraphExec_t x = nullptr;
        if (cudaGraphInstantiate(&x, g, 0) != cudaSuccess || !x) {
            cudaGraphDestroy(g);
            note_failure("instantiate");
            return;
        }
        cudaGraphGetNodes(g, nullptr, &nodes_);
        graph_ = g;
        exec_ = x;
    }
    void note_failure(const char* what) {
        const cudaError_t e = cudaGetLastError();   // clears the sticky slot for the fallback
        if (what) last_error_ = std::string(what) + ": " + cudaGetErrorString(e);
        ++failures_;
    }
    cudaGraph_t graph_ = nullptr;
    cudaGraphExec_t exec_ = nullptr;
    size_t nodes_ = 0;
    uint64_t replays_ = 0;
    int failures_ = 0, give_up_after_;
    std::string last_error_;
};

// ---------------------------------------------------------------------------
// The loop itself.
// ---------------------------------------------------------------------------
struct DecodeLoopConfig {
    uint32_t layers = 0, batch = 1, heads = 0, kv_heads = 0, head_dim = 0, max_seq_len = 2048;
    int32_t window = 0;     // sliding window of every layer (0 = all positions)
    float scale = 0.0f;     // 0 = 1/sqrt(head_dim), the reference's default (src/command.cpp:160)
};

// One layer of a model whose layers differ (reference src/graph_builder.cpp:692-778, the Gemma-4
// emission): its own head_dim, its own window (`window = is_global ? 0 : sliding_window`, :699), its
// own softmax scale (Gemma-4 passes 1.0, :767/:777), its own plane — which a shared layer borrows
// from an earlier owner and must not append to (:746).
struct DecodeLayer {
    uint32_t head_dim = 0;
    uint32_t rows = 0;          // rows per sequence of the plane (max_seq_len, or the ring size)
    int32_t window = 0;         // 0 = attend everything
    int32_t layout = HKV_LAYOUT_LINEAR;
    bool append = true;         // false: shared layer, attends an owner's plane, writes nothing
    float scale = 0.0f;         // 0 = 1/sqrt(head_dim)
    half* k_plane = nullptr;    // [batch][rows][kv_heads][head_dim], owned by the caller's cache
    half* v_plane = nullptr;
};

// The per-layer plan of a Gemma4KVCache: owners append, shared layers only attend; local layers
// take their sliding window (over a ring plane when the cache was allocated with one).
inline std::vector<DecodeLayer> decode_layers_of(Gemma4KVCache& cache, float scale) {
    std::vector<DecodeLayer> out(cache.num_layers());
    for (uint32_t l = 0; l < cache.num_layers(); ++l) {
        DecodeLayer& d = out[l];
        d.head_dim = cache.head_dim(l);
        d.rows = cache.rows(l);
        d.window = cache.is_global(l) ? 0 : (int32_t)cache.sliding_window(l);
        d.layout = cache.is_ring(l) ? HKV_LAYOUT_RING : HKV_LAYOUT_LINEAR;
        d.append = !cache.is_shared(l);
        d.scale = scale;
        d.k_plane = cache.k_cache(l);
        d.v_plane = cache.v_cache(l);
    }
    return out;
}

class BatchedDecodeLoop {
public:
    // Called before each layer's attention is enqueued: the place for the model's other ops of
    // that layer (they land in the same captured graph). May be empty.
    using LayerHook = std::function<void(uint32_t layer, cudaStream_t stream)>;

    // Every layer alike; the loop owns the planes.
    BatchedDecodeLoop(const DecodeLoopConfig& cfg, cudaStream_t stream)
        : cfg_(cfg), stream_(stream), board_(cfg.batch, cfg.max_seq_len) {
        KVCacheConfig kc;
        kc.num_layers = cfg.layers; kc.num_kv_heads = cfg.kv_heads; kc.head_dim = cfg.head_dim;
        kc.max_batch_size = cfg.batch; kc.max_seq_len = cfg.max_seq_len;
        if (!cache_.allocate(kc)) throw std::runtime_error("BatchedDecodeLoop: cache allocation failed");
        std::vector<DecodeLayer> layers(cfg.layers);
        for (uint32_t l = 0; l < cfg.layers; ++l) {
            layers[l].head_dim = cfg.head_dim; layers[l].rows = cfg.max_seq_len; layers[l].window = cfg.window;
            layers[l].scale = cfg.scale; layers[l].k_plane = cache_.k_cache(l); layers[l].v_plane = cache_.v_cache(l);
        }
        set_layers(std::move(layers));
    }
    // Layers that differ (head_dim, window, ring or linear plane, scale, shared or owner); the planes
    // belong to the caller's cache object (e.g. Gemma4KVCache + decode_layers_of) and must outlive
    // the loop. `max_seq_len` bounds the positions a session can reach.
    BatchedDecodeLoop(uint32_t batch, uint32_t heads, uint32_t kv_heads, uint32_t max_seq_len,
                      std::vector<DecodeLayer> layers, cudaStream_t stream)
        : stream_(stream), board_(batch, max_seq_len) {
        cfg_.layers = (uint32_t)layers.size(); cfg_.batch = batch; cfg_.heads = heads; cfg_.kv_heads = kv_heads;
        cfg_.max_seq_len = max_seq_len;
        set_layers(std::move(layers));
    }
    ~BatchedDecodeLoop() {
        graph_.invalidate();
        for (auto& kv : ctxs_) hkv_ctx_destroy(kv.second);
    }
    BatchedDecodeLoop(const BatchedDecodeLoop&) = delete;
    BatchedDecodeLoop& operator=(const BatchedDecodeLoop&) = delete;

    SessionBoard& board() { return board_; }
    KVCache& cache() { return cache_; }
    GraphReplay& graph() { return graph_; }
    hkv_ctx* context(uint32_t layer = 0) { return layer < layer_ctx_.size() ? layer_ctx_[layer] : nullptr; }
    size_t contexts() const { return ctxs_.size(); }
    const DecodeLoopConfig& config() const { return cfg_; }
    const std::vector<DecodeLayer>& layers() const { return layers_; }
    // Element offsets of layer l inside the bound activation buffers (layers may differ in head_dim).
    size_t q_offset(uint32_t layer) const { return q_off_[layer]; }
    size_t kv_offset(uint32_t layer) const { return kv_off_[layer]; }
    size_t q_elems() const { return q_off_.back(); }
    size_t kv_elems() const { return kv_off_.back(); }

    // Binds the activation buffers the graph reads and writes; they must keep their addresses for
    // as long as the graph lives (rebinding drops the graph). Layer l uses
    //   q + q_offset(l) [batch][heads][head_dim(l)], out likewise,
    //   k_new / v_new + kv_offset(l) [batch][kv_heads][head_dim(l)] (never read for a shared layer).
    // With every layer alike these are the plain strides l*batch*heads*head_dim and l*batch*kv_heads*head_dim.
    void bind(const half* q, const half* k_new, const half* v_new, half* out, LayerHook hook = nullptr) {
        q_ = q; k_new_ = k_new; v_new_ = v_new; out_ = out; hook_ = std::move(hook);
        graph_.invalidate();
    }

    // One token for every active session: publish positions, run all layers, advance. Returns
    // true when the step was a graph replay. Nothing here synchronises with the device.
    bool step() {
        if (!q_ || !k_new_ || !v_new_ || !out_) throw std::runtime_error("BatchedDecodeLoop: bind() first");
        board_.publish(stream_, 1);
        const bool replayed = graph_.run(stream_, [this](cudaStream_t s) { enqueue_layers(s); });
        board_.advance_all(1);
        ++tokens_;
        return replayed;
    }
    uint64_t steps() const { return tokens_; }
    // Device-side status words of all contexts OR-ed (a bounded wait that ran out, etc.); synchronises.
    int device_status() {
        int32_t all = 0;
        for (auto& kv : ctxs_) { int32_t w = 0; hkv_ctx_device_status(kv.second, stream_, &w); all |= w; }
        return all;
    }

private:
    using CtxKey = std::tuple<uint32_t, uint32_t, int32_t, int32_t>;   // head_dim, rows, window, layout
    void set_layers(std::vector<DecodeLayer> layers) {
        if (layers.empty()) throw std::runtime_error("BatchedDecodeLoop: no layers");
        layers_ = std::move(layers);
        q_off_.assign(1, 0);
        kv_off_.assign(1, 0);
        for (DecodeLayer& d : layers_) {
            if (!d.head_dim || !d.rows || !d.k_plane || !d.v_plane) throw std::runtime_error("BatchedDecodeLoop: incomplete layer");
            if (d.scale == 0.0f) d.scale = 1.0f / std::sqrt((float)d.head_dim);
            const CtxKey key{d.head_dim, d.rows, d.window, d.layout};
            auto it = ctxs_.find(key);
            if (it == ctxs_.end()) {   // one context per distinct layer geometry; allocates: before any capture
                hkv_geometry g{};
                g.batch = (int32_t)cfg_.batch; g.num_heads = (int32_t)cfg_.heads; g.num_kv_heads = (int32_t)cfg_.kv_heads;
                g.head_dim = (int32_t)d.head_dim; g.slots = (int32_t)d.rows; g.window_size = d.window; g.layout = d.layout;
                hkv_ctx* c = nullptr;
                const int st = hkv_ctx_create(&c, &g);
                if (st != HKV_OK) {
                    std::string msg = std::string("BatchedDecodeLoop: hkv_ctx_create: ") + hkv_status_string(st);
                    if (c) { msg += std::string(" (") + hkv_ctx_last_error(c) + ")"; hkv_ctx_destroy(c); }
                    throw std::runtime_error(msg);
                }
                it = ctxs_.emplace(key, c).first;
            }
            layer_ctx_.push_back(it->second);
            q_off_.push_back(q_off_.back() + (size_t)cfg_.batch * cfg_.heads * d.head_dim);
            kv_off_.push_back(kv_off_.back() + (size_t)cfg_.batch * cfg_.kv_heads * d.head_dim);
        }
    }
    void enqueue_layers(cudaStream_t s) {
        for (uint32_t l = 0; l < (uint32_t)layers_.size(); ++l) {
            if (hook_) hook_(l, s);
            const DecodeLayer& d = layers_[l];
            hkv_ctx* c = layer_ctx_[l];
            // owner: fused append + attention at the device position; shared layer: attention only,
            // over the plane its owner has already appended this token's row to
            const int st = d.append
                               ? hkv_append_decode_attention(c, q_ + q_off_[l], k_new_ + kv_off_[l], v_new_ + kv_off_[l], d.k_plane,
                                                             d.v_plane, out_ + q_off_[l], board_.d_cache_pos(), d.scale, s)
                               : hkv_decode_attention(c, q_ + q_off_[l], d.k_plane, d.v_plane, out_ + q_off_[l],
                                                      board_.d_total_seq(), d.scale, s);
            if (st != HKV_OK)
                throw std::runtime_error(std::string("BatchedDecodeLoop: layer ") + std::to_string(l) + ": " +
                                         hkv_ctx_last_error(c));
        }
    }
    DecodeLoopConfig cfg_;
    cudaStream_t stream_;
    SessionBoard board_;
    KVCache cache_;                       // used by the uniform constructor only
    GraphReplay graph_;
    std::vector<DecodeLayer> layers_;
    std::map<CtxKey, hkv_ctx*> ctxs_;
    std::vector<hkv_ctx*> layer_ctx_;
    std::vector<size_t> q_off_, kv_off_;
    const half* q_ = nullptr;
    const half* k_new_ = nullptr;
    const half* v_new_ = nullptr;
    half* out_ = nullptr;
    LayerHook hook_;
    uint64_t tokens_ = 0;
};

}  // namespace hkv
