// hkv_register.hpp — registers libhkv's ops into a host engine at its kernel-registry
// boundary, in place of the engine's own attention ops.
//
// The three lambdas keep the reference ops' contract (reference project paths):
//   ATTENTION_CACHED           kernels/register_kernels.cpp:841-887
//   ATTENTION_PREFILL_CACHED   kernels/register_kernels.cpp:891-921
//   KV_CACHE_UPDATE            kernels/register_kernels.cpp:924-980
//   QK_NORM_ROPE               kernels/register_kernels.cpp:777-837 (the step in front of the append)
// i.e. the same input order, parameter keys and defaults, the same geometry guard and
// dtype check, std::runtime_error for every failure, work enqueued only on ctx.stream.
// ATTENTION_CACHED additionally accepts the five-input form (Q, K_cache, V_cache, K_new,
// V_new) that the op registry declares (src/optype.cpp:118-120): append + attention fused.
//
// `Bind` adapts the adapter to an engine's types. For the reference engine:
//
//   struct HeliosBind {
//       using Engine = helios::Engine;  using ExecContext = helios::ExecContext;
//       using Command = helios::Command; using TensorInfo = helios::TensorInfo;
//       static uint32_t attention_cached()         { return helios::op::ATTENTION_CACHED(); }
//       static uint32_t kv_cache_update()          { return helios::op::KV_CACHE_UPDATE(); }
//       static uint32_t attention_prefill_cached() { return helios::op::ATTENTION_PREFILL_CACHED(); }
//       static uint32_t qk_norm_rope()             { return helios::op::QK_NORM_ROPE(); }
//       static bool is_fp16(const TensorInfo& t)   { return t.dtype == helios::dtype::FP16(); }
//       static const char* dtype_name(const TensorInfo& t) { return helios::dtype_name(t.dtype); }
//   };
//   hkv::Registration<HeliosBind> ops(engine);   // after kernels::register_all_kernels(engine)
#pragma once

#include <cmath>
#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>

#include "hkv.h"

namespace hkv {

// Owns one hkv_ctx per distinct geometry; turns status codes into exceptions.
class ContextPool {
public:
    ContextPool() = default;
    ~ContextPool();
    ContextPool(const ContextPool&) = delete;
    ContextPool& operator=(const ContextPool&) = delete;

    // Returns the context for this geometry, creating it on first use. Creation allocates,
    // so the first use of a geometry must happen outside stream capture (the engine runs
    // the first token un-captured); prepare() does it explicitly at model load.
    hkv_ctx* get(const hkv_geometry& g);
    void prepare(const hkv_geometry& g) { (void)get(g); }
    size_t size() const { return ctxs_.size(); }
    static void check(hkv_ctx* c, int status, const char* op);

private:
    using Key = std::tuple<int, int, int, int, int, int, int, long long, int, int>;
    std::map<Key, hkv_ctx*> ctxs_;
};

template <class Bind>
class Registration {
public:
    using Engine = typename Bind::Engine;
    using ExecContext = typename Bind::ExecContext;
    using Command = typename Bind::Command;
    using TensorInfo = typename Bind::TensorInfo;

    explicit Registration(Engine& engine) : engine_(engine), pool_(std::make_shared<ContextPool>()) {
        auto pool = pool_;
        Engine* eng = &engine;

        engine.register_kernel(Bind::attention_cached(), [pool, eng](ExecContext& ctx, const Command& cmd) {
            TensorInfo* q = ctx.in(0);
            TensorInfo* k_cache = ctx.in(1);
            TensorInfo* v_cache = ctx.in(2);
            TensorInfo* output = ctx.output;
            if (!q || !k_cache || !v_cache || !output)
                throw std::runtime_error("ATTENTION_CACHED: missing tensors");
            const bool fused = ctx.num_inputs() >= 5;
            TensorInfo* k_new = fused ? ctx.in(3) : nullptr;
            TensorInfo* v_new = fused ? ctx.in(4) : nullptr;
            if (fused && (!k_new || !v_new))
                throw std::runtime_error("ATTENTION_CACHED: missing K_new/V_new tensors");

            const uint32_t num_heads = cmd.template get<uint32_t>("num_heads", 32);
            const uint32_t num_kv_heads = cmd.template get<uint32_t>("num_kv_heads", num_heads);
            const uint32_t head_dim = cmd.template get<uint32_t>("head_dim", 128);
            const float scale = cmd.template get<float>("scale", 1.0f / std::sqrt(float(head_dim)));
            const uint32_t seq_len = cmd.template get<uint32_t>("seq_len", 1);
            const uint32_t max_seq_len = cmd.template get<uint32_t>("max_seq_len", 2048);
            const uint32_t window_size = cmd.template get<uint32_t>("window_size", 0);
            if (head_dim == 0 || head_dim > 512 || num_kv_heads == 0 || num_heads == 0 ||
                num_heads % num_kv_heads != 0)
                throw std::runtime_error("ATTENTION_CACHED: unsupported head geometry");

            hkv_geometry g = geometry(1, num_heads, num_kv_heads, head_dim, max_seq_len, window_size);
            hkv_ctx* c = pool->get(g);
            const bool dev_pos = cmd.template get<uint32_t>("device_pos", 0) && eng->has_device_cache_pos();
            if (fused) {
                if (!dev_pos)
                    throw std::runtime_error("ATTENTION_CACHED: the fused five-input form needs device_pos");
                ContextPool::check(c, hkv_append_decode_attention(c, fp16(q), fp16(k_new), fp16(v_new),
                                                                  fp16(k_cache), fp16(v_cache), fp16(output),
                                                                  eng->device_cache_pos(), scale, ctx.stream),
                                   "ATTENTION_CACHED");
            } else if (dev_pos) {
                ContextPool::check(c, hkv_decode_attention(c, fp16(q), fp16(k_cache), fp16(v_cache), fp16(output),
                                                           eng->device_total_seq(), scale, ctx.stream),
                                   "ATTENTION_CACHED");
            } else {
                ContextPool::check(c, hkv_decode_attention_len(c, fp16(q), fp16(k_cache), fp16(v_cache),
                                                               fp16(output), (int32_t)seq_len, scale, ctx.stream),
                                   "ATTENTION_CACHED");
            }
        });

        engine.register_kernel(Bind::attention_prefill_cached(), [pool](ExecContext& ctx, const Command& cmd) {
            TensorInfo* q = ctx.in(0);
            TensorInfo* k_cache = ctx.in(1);
            TensorInfo* v_cache = ctx.in(2);
            TensorInfo* output = ctx.output;
            if (!q || !k_cache || !v_cache || !output)
                throw std::runtime_error("ATTENTION_PREFILL_CACHED: missing tensors");
            const uint32_t num_heads = cmd.template get<uint32_t>("num_heads", 32);
            const uint32_t num_kv_heads = cmd.template get<uint32_t>("num_kv_heads", num_heads);
            const uint32_t head_dim = cmd.template get<uint32_t>("head_dim", 128);
            const float scale = cmd.template get<float>("scale", 1.0f / std::sqrt(float(head_dim)));
            const uint32_t seq_new = cmd.template get<uint32_t>("seq_len", 1);
            const uint32_t past_len = cmd.template get<uint32_t>("past_len", 0);
            const uint32_t max_seq_len = cmd.template get<uint32_t>("max_seq_len", 2048);
            const uint32_t window_size = cmd.template get<uint32_t>("window_size", 0);
            if (head_dim == 0 || head_dim > 512 || num_kv_heads == 0 || num_heads == 0 ||
                num_heads % num_kv_heads != 0)
                throw std::runtime_error("ATTENTION_PREFILL_CACHED: unsupported head geometry");
            hkv_geometry g = geometry(1, num_heads, num_kv_heads, head_dim, max_seq_len, window_size);
            // Chunks may be cut by key range to fill the SMs (the engine's chunk of 512 queries makes
            // fewer work items than a B200 has SMs), which needs a workspace of partials sized by the
            // chunk. The size is rounded up to 512, 1024, 2048 or 4096 so that ragged chunks share a
            // context and at most four exist per geometry; longer chunks have enough work items
            // without a split and get none.
            g.max_seq_new = 0;
            for (uint32_t cap = 512; cap <= 4096; cap *= 2)
                if (seq_new <= cap) { g.max_seq_new = (int32_t)cap; break; }
            hkv_ctx* c = pool->get(g);
            ContextPool::check(c, hkv_prefill_attention(c, fp16(q), fp16(k_cache), fp16(v_cache), fp16(output),
                                                        (int32_t)seq_new, (int32_t)past_len, scale, ctx.stream),
                               "ATTENTION_PREFILL_CACHED");
        });

        // QK_NORM_ROPE (kernels/register_kernels.cpp:777-837): inputs q, k, q_norm_w, k_norm_w and,
        // in the fused form, v, k_cache, v_cache; the fused form also writes the cache.
        engine.register_kernel(Bind::qk_norm_rope(), [pool, eng](ExecContext& ctx, const Command& cmd) {
            TensorInfo* q = ctx.in(0);
            TensorInfo* k = ctx.in(1);
            TensorInfo* qw = ctx.in(2);
            TensorInfo* kw = ctx.in(3);
            if (!q || !k || !qw || !kw) throw std::runtime_error("QK_NORM_ROPE: missing tensors");
            const uint32_t H = cmd.template get<uint32_t>("num_heads", 32);
            const uint32_t KVH = cmd.template get<uint32_t>("num_kv_heads", H);
            const uint32_t HD = cmd.template get<uint32_t>("dim", 128);
            const uint32_t seq_len = cmd.template get<uint32_t>("seq_len", 1);
            const uint32_t offset = cmd.template get<uint32_t>("offset", 0);
            const float eps = cmd.template get<float>("eps", 1e-6f);
            const float theta = cmd.template get<float>("theta", 10000.0f);
            const float partial_rotary = cmd.template get<float>("partial_rotary", 1.0f);
            const float scaling_factor = cmd.template get<float>("rope_scaling_factor", 1.0f);
            int rotary_dim = (int)(HD * partial_rotary);
            rotary_dim = (rotary_dim / 2) * 2;
            if (rotary_dim <= 0) rotary_dim = (int)HD;
            if (HD == 0 || HD > 512 || KVH == 0 || H == 0 || H % KVH != 0)
                throw std::runtime_error("QK_NORM_ROPE: unsupported head geometry");
            const bool dev_pos = cmd.template get<uint32_t>("device_pos", 0) && eng->has_device_cache_pos();
            const uint32_t max_seq_len = cmd.template get<uint32_t>("max_seq_len", 4096);
            hkv_geometry g = geometry(1, H, KVH, HD, max_seq_len, 0);
            g.flags = HKV_FLAG_APPEND_ONLY;   // norm + rope + cache write: no attention workspace
            hkv_ctx* c = pool->get(g);
            void *v = nullptr, *kc = nullptr, *vc = nullptr;
            if (ctx.num_inputs() >= 7) {
                TensorInfo* tv = ctx.in(4);
                TensorInfo* tkc = ctx.in(5);
                TensorInfo* tvc = ctx.in(6);
                if (!tv || !tkc || !tvc) throw std::runtime_error("QK_NORM_ROPE: missing kv cache tensors");
                v = fp16(tv);
                kc = fp16(tkc);
                vc = fp16(tvc);
            }
            ContextPool::check(c, hkv_qk_norm_rope_kv(c, fp16(q), fp16(k), v, fp16(qw), fp16(kw), kc, vc,
                                                      dev_pos ? eng->device_cache_pos() : nullptr, (int32_t)offset,
                                                      (int32_t)seq_len, rotary_dim, eps, theta, scaling_factor,
                                                      ctx.stream),
                               "QK_NORM_ROPE");
        });

        engine.register_kernel(Bind::kv_cache_update(), [pool, eng](ExecContext& ctx, const Command& cmd) {
            TensorInfo* k_new = ctx.in(0);
            TensorInfo* v_new = ctx.in(1);
            TensorInfo* k_cache = ctx.in(2);
            TensorInfo* v_cache = ctx.in(3);
            if (!k_new || !v_new || !k_cache || !v_cache)
                throw std::runtime_error("KV_CACHE_UPDATE: missing tensors");
            const uint32_t position = cmd.template get<uint32_t>("position", 0);
            const uint32_t max_seq_len = cmd.template get<uint32_t>("max_seq_len", 2048);
            const uint32_t kv_heads = cmd.template get<uint32_t>("num_kv_heads", 2);
            const uint32_t head_dim = cmd.template get<uint32_t>("head_dim", 128);
            if (head_dim == 0 || head_dim > 512 || kv_heads == 0)
                throw std::runtime_error("KV_CACHE_UPDATE: unsupported head geometry");
            // seq_len from the command when given (scratch tensors are oversized), else from the shape
            int batch = 1;
            int seq_len = (int)cmd.template get<uint32_t>("seq_len", 0u);
            if (seq_len == 0) {
                if (k_new->shape.size() >= 3) {
                    batch = (int)k_new->shape[0];
                    seq_len = (int)k_new->shape[1];
                } else if (k_new->shape.size() == 2) {
                    const int total = (int)(k_new->size_bytes / 2);
                    seq_len = total / (int)(kv_heads * head_dim * batch);
                    if (seq_len < 1) seq_len = 1;
                }
            } else if (k_new->shape.size() >= 3) {
                batch = (int)k_new->shape[0];
            }
            hkv_geometry g = geometry(batch, kv_heads, kv_heads, head_dim, max_seq_len, 0);
            // The engine's device position is ONE scalar that every sequence of the batch writes at
            // (kernels/register_kernels.cpp:959-968 forwards `batch` with it): same here.
            g.flags = HKV_FLAG_APPEND_ONLY | HKV_FLAG_SCALAR_POSITION;
            hkv_ctx* c = pool->get(g);
            if (cmd.template get<uint32_t>("device_pos", 0) && eng->has_device_cache_pos()) {
                ContextPool::check(c, hkv_append(c, fp16(k_new), fp16(v_new), fp16(k_cache), fp16(v_cache),
                                                 eng->device_cache_pos(), seq_len, ctx.stream),
                                   "KV_CACHE_UPDATE");
            } else {
                ContextPool::check(c, hkv_append_at(c, fp16(k_new), fp16(v_new), fp16(k_cache), fp16(v_cache),
                                                    (int32_t)position, seq_len, ctx.stream),
                                   "KV_CACHE_UPDATE");
            }
        });
    }

    // Allocate the context of a geometry ahead of time (outside capture).
    void prepare(int batch, uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim,
                 uint32_t max_seq_len, uint32_t window_size) {
        pool_->prepare(geometry(batch, num_heads, num_kv_heads, head_dim, max_seq_len, window_size));
    }
    size_t contexts() const { return pool_->size(); }

private:
    static hkv_geometry geometry(int batch, uint32_t H, uint32_t KVH, uint32_t HD, uint32_t max_seq,
                                 uint32_t window) {
        hkv_geometry g{};
        g.batch = batch;
        g.num_heads = (int32_t)H;
        g.num_kv_heads = (int32_t)KVH;
        g.head_dim = (int32_t)HD;
        g.slots = (int32_t)max_seq;
        g.window_size = (int32_t)window;
        g.layout = HKV_LAYOUT_LINEAR;
        return g;
    }
    // Typed pointer with the engine's dtype check (kernels/register_kernels.cpp:22-42).
    static void* fp16(TensorInfo* t) {
        if (!Bind::is_fp16(*t))
            throw std::runtime_error(std::string("Expected FP16 tensor but got ") + Bind::dtype_name(*t) +
                                     " — check model dtype vs kernel dispatch");
        return t->ptr;
    }

    Engine& engine_;
    std::shared_ptr<ContextPool> pool_;
};

}  // namespace hkv
