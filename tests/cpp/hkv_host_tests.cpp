// hkv_host_tests.cpp — C++ tests of the registry-boundary adapter (hkv_register.hpp) driven
// through the engine shim, checked against the CPU oracle. Needs a B200; `--list` does not.
//
// Cases: the reference's known-answer vectors (reference tests/test_gemma4_kv.cu:234-347)
// issued as command buffers; the CUDA-graph capture-once contract (capture on the second
// token, replay while only the device position changes — reference src/engine.cpp:151-269);
// the fused five-input op; the ops' error behaviour; the C++ cache owner.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "hkv.h"
#include "hkv_engine_shim.hpp"
#include "hkv_decode_loop.hpp"
#include "hkv_kv_cache.hpp"
#include "hkv_register.hpp"

extern "C" {
uint16_t hkv_oracle_f2h(float f);
float hkv_oracle_h2f(uint16_t h);
void hkv_oracle_fill(uint16_t* dst, uint64_t seed, uint64_t first_index, uint64_t count);
void hkv_oracle_append(const uint16_t* new_k, const uint16_t* new_v, uint16_t* k_cache, uint16_t* v_cache,
                       int B, int S, int KVH, int HD, int slots, int64_t batch_stride, const int32_t* pos,
                       int layout);
void hkv_oracle_decode(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out,
                       float* out_f32, int B, const int32_t* total, int H, int KVH, int HD, int slots,
                       int64_t batch_stride, float scale, int window, int layout, int mode, int threads);
void hkv_oracle_qk_norm_rope(uint16_t* q, uint16_t* k, const uint16_t* v, const uint16_t* q_w, const uint16_t* k_w,
                             uint16_t* k_cache, uint16_t* v_cache, int B, int S, int H, int KVH, int HD,
                             int rotary_dim, const int32_t* pos, int slots, int layout, float eps, float theta,
                             float scaling);
}

namespace sh = hkv_shim;

struct ShimBind {
    using Engine = sh::Engine;
    using ExecContext = sh::ExecContext;
    using Command = sh::Command;
    using TensorInfo = sh::TensorInfo;
    static uint32_t attention_cached() { return sh::op::ATTENTION_CACHED(); }
    static uint32_t kv_cache_update() { return sh::op::KV_CACHE_UPDATE(); }
    static uint32_t attention_prefill_cached() { return sh::op::ATTENTION_PREFILL_CACHED(); }
    static uint32_t qk_norm_rope() { return sh::op::QK_NORM_ROPE(); }
    static bool is_fp16(const TensorInfo& t) { return t.dtype == sh::DType::FP16; }
    static const char* dtype_name(const TensorInfo& t) { return sh::dtype_name(t.dtype); }
};

static int g_failures = 0;
#define REQUIRE(cond, msg)                                              \
    do {                                                                \
        if (!(cond)) {                                                  \
            std::printf("FAIL: %s (%s:%d)\n", msg, __FILE__, __LINE__); \
            ++g_failures;                                               \
            return;                                                     \
        }                                                               \
    } while (0)

static std::vector<uint16_t> halves(size_t n, float v) { return std::vector<uint16_t>(n, hkv_oracle_f2h(v)); }
static void upload(void* dst, const std::vector<uint16_t>& src, cudaStream_t st = nullptr) {
    cudaMemcpyAsync(dst, src.data(), src.size() * 2, cudaMemcpyHostToDevice, st);
    cudaStreamSynchronize(st);
}
static std::vector<uint16_t> download(const void* src, size_t n) {
    std::vector<uint16_t> out(n);
    cudaMemcpy(out.data(), src, n * 2, cudaMemcpyDeviceToHost);
    return out;
}
static bool close_enough(const std::vector<uint16_t>& got, const std::vector<uint16_t>& ref, float* worst) {
    *worst = 0.0f;
    for (size_t i = 0; i < got.size(); ++i) {
        const float x = hkv_oracle_h2f(got[i]), r = hkv_oracle_h2f(ref[i]);
        const float err = std::fabs(x - r);
        if (err > *worst) *worst = err;
        if (!(err <= 2e-3f + 1e-2f * std::fabs(r))) return false;  // the path's tolerance
    }
    return true;
}

// ---------------------------------------------------------------------------
static void test_known_answers() {
    sh::Engine engine;
    hkv::Registration<ShimBind> ops(engine);
    auto& T = engine.tensors();
    // decode, window 3 of 6 positions: mean of V = 4, 5, 6
    T.allocate_and_register("attn.q", {1, 1, 1, 2}, sh::DType::FP16);
    T.allocate_and_register("attn.k", {1, 6, 1, 2}, sh::DType::FP16);
    T.allocate_and_register("attn.v", {1, 6, 1, 2}, sh::DType::FP16);
    T.allocate_and_register("attn.out", {1, 1, 1, 2}, sh::DType::FP16);
    std::vector<uint16_t> v(12);
    for (int p = 0; p < 6; ++p) v[p * 2] = v[p * 2 + 1] = hkv_oracle_f2h(float(p + 1));
    upload(T.at("attn.v").ptr, v);
    sh::CommandBuffer local;
    local.add_attention_cached("attn.out", "attn.q", "attn.k", "attn.v", 1, 1, 2, 6, 6, 3);
    engine.execute(local);
    engine.sync();
    auto out = download(T.at("attn.out").ptr, 2);
    REQUIRE(std::fabs(hkv_oracle_h2f(out[0]) - 5.0f) < 0.01f && std::fabs(hkv_oracle_h2f(out[1]) - 5.0f) < 0.01f,
            "decode local mask keeps only the last three values");

    // prefill, 2 new queries after 4 cached positions, window 3
    T.allocate_and_register("prefill.q", {1, 2, 1, 2}, sh::DType::FP16);
    T.allocate_and_register("prefill.out", {1, 2, 1, 2}, sh::DType::FP16);
    sh::CommandBuffer prefill;
    prefill.add_op(sh::op::ATTENTION_PREFILL_CACHED(), "prefill.out")
        .in({"prefill.q", "attn.k", "attn.v"})
        .set("num_heads", uint32_t{1}).set("num_kv_heads", uint32_t{1}).set("head_dim", uint32_t{2})
        .set("scale", 1.0f).set("seq_len", uint32_t{2}).set("past_len", uint32_t{4})
        .set("max_seq_len", uint32_t{6}).set("window_size", uint32_t{3});
    engine.execute(prefill);
    engine.sync();
    auto pout = download(T.at("prefill.out").ptr, 4);
    REQUIRE(std::fabs(hkv_oracle_h2f(pout[0]) - 4.0f) < 0.01f && std::fabs(hkv_oracle_h2f(pout[2]) - 5.0f) < 0.01f,
            "prefill local mask slides independently for each new query");

    // 514 positions, window 512: the first two rows (V = 1000) are excluded
    T.allocate_and_register("boundary.k", {1, 514, 1, 2}, sh::DType::FP16);
    T.allocate_and_register("boundary.v", {1, 514, 1, 2}, sh::DType::FP16);
    T.allocate_and_register("boundary.out", {1, 1, 1, 2}, sh::DType::FP16);
    auto bv = halves(514 * 2, 2.0f);
    for (int i = 0; i < 4; ++i) bv[i] = hkv_oracle_f2h(1000.0f);
    upload(T.at("boundary.v").ptr, bv);
    sh::CommandBuffer boundary;
    boundary.add_attention_cached("boundary.out", "attn.q", "boundary.k", "boundary.v", 1, 1, 2, 514, 514, 512);
    engine.execute(boundary);
    engine.sync();
    auto bout = download(T.at("boundary.out").ptr, 2);
    REQUIRE(std::fabs(hkv_oracle_h2f(bout[0]) - 2.0f) < 0.01f, "token 514 excludes the two rows outside the 512 window");

    // head_dim 512, two positions V = 2 and 6 -> every dimension 4
    T.allocate_and_register("global.q", {1, 1, 1, 512}, sh::DType::FP16);
    T.allocate_and_register("global.k", {1, 2, 1, 512}, sh::DType::FP16);
    T.allocate_and_register("global.v", {1, 2, 1, 512}, sh::DType::FP16);
    T.allocate_and_register("global.out", {1, 1, 1, 512}, sh::DType::FP16);
    auto gv = halves(1024, 2.0f);
    for (size_t i = 512; i < 1024; ++i) gv[i] = hkv_oracle_f2h(6.0f);
    upload(T.at("global.v").ptr, gv);
    sh::CommandBuffer global;
    global.add_attention_cached("global.out", "global.q", "global.k", "global.v", 1, 1, 512, 2, 2);
    engine.execute(global);
    engine.sync();
    auto gout = download(T.at("global.out").ptr, 512);
    for (uint16_t h : gout) REQUIRE(std::fabs(hkv_oracle_h2f(h) - 4.0f) < 0.01f, "HD512 writes every dimension");
    std::printf("PASS: known answers (decode window, prefill window, >512 boundary, HD512)\n");
}

// ---------------------------------------------------------------------------
// Capture once, replay while only the device position changes; fused = five-input op.
static void run_graph_contract(bool fused) {
    const int H = 14, KVH = 2, HD = 64, S = 2048;
    cudaStream_t stream;
    cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);  // capture needs a non-legacy stream
    {
        sh::Engine engine(stream);
        hkv::Registration<ShimBind> ops(engine);
        engine.alloc_device_cache_pos();
        auto& T = engine.tensors();
        T.allocate_and_register("q", {1, 1, (uint32_t)H, (uint32_t)HD}, sh::DType::FP16);
        T.allocate_and_register("k_new", {1, 1, (uint32_t)(KVH * HD)}, sh::DType::FP16);
        T.allocate_and_register("v_new", {1, 1, (uint32_t)(KVH * HD)}, sh::DType::FP16);
        T.allocate_and_register("kc", {1, (uint32_t)S, (uint32_t)KVH, (uint32_t)HD}, sh::DType::FP16);
        T.allocate_and_register("vc", {1, (uint32_t)S, (uint32_t)KVH, (uint32_t)HD}, sh::DType::FP16);
        T.allocate_and_register("out", {1, 1, (uint32_t)H, (uint32_t)HD}, sh::DType::FP16);

        const int start = 500, steps = 24;
        const size_t row = (size_t)KVH * HD;
        std::vector<uint16_t> hk((size_t)S * row, 0), hv((size_t)S * row, 0);
        hkv_oracle_fill(hk.data(), 11, 0, (uint64_t)start * row);
        hkv_oracle_fill(hv.data(), 12, 0, (uint64_t)start * row);
        upload(T.at("kc").ptr, hk, stream);
        upload(T.at("vc").ptr, hv, stream);

        sh::CommandBuffer cb;
        if (fused) {
            cb.add_op(sh::op::ATTENTION_CACHED(), "out")
                .in({"q", "kc", "vc", "k_new", "v_new"})
                .set("num_heads", uint32_t(H)).set("num_kv_heads", uint32_t(KVH)).set("head_dim", uint32_t(HD))
                .set("max_seq_len", uint32_t(S)).set("device_pos", uint32_t{1});
        } else {
            cb.add_kv_cache_update("kc", "vc", "k_new", "v_new", 0, S, KVH, HD, 1);
            cb.commands().back().set("device_pos", uint32_t{1});
            cb.add_attention_cached("out", "q", "kc", "vc", H, KVH, HD, 1, S, 0);
            cb.commands().back().set("device_pos", uint32_t{1});
        }

        const float scale = 1.0f / std::sqrt(float(HD));
        size_t ctx_after_first = 0;
        for (int s = 0; s < steps; ++s) {
            const int pos = start + s;
            std::vector<uint16_t> q((size_t)H * HD), nk(row), nv(row);
            hkv_oracle_fill(q.data(), 100 + s, 0, q.size());
            hkv_oracle_fill(nk.data(), 200 + s, 0, row);
            hkv_oracle_fill(nv.data(), 300 + s, 0, row);
            upload(T.at("q").ptr, q, stream);  // same device addresses every step
            upload(T.at("k_new").ptr, nk, stream);
            upload(T.at("v_new").ptr, nv, stream);
            engine.update_device_cache_pos(pos, 1);
            if (s == 0) {
                engine.execute(cb);  // first token un-captured: contexts are created here
                ctx_after_first = ops.contexts();
            } else {
                const bool graphed = engine.execute_graph_replay(cb);
                REQUIRE(graphed, engine.last_capture_error().c_str());
            }
            engine.sync();
            // oracle mirror
            const int32_t p32 = pos, tot = pos + 1;
            hkv_oracle_append(nk.data(), nv.data(), hk.data(), hv.data(), 1, 1, KVH, HD, S, 0, &p32, 0);
            std::vector<uint16_t> ref((size_t)H * HD);
            hkv_oracle_decode(q.data(), hk.data(), hv.data(), ref.data(), nullptr, 1, &tot, H, KVH, HD, S, 0,
                              scale, 0, 0, 0, 1);
            float worst;
            REQUIRE(close_enough(download(T.at("out").ptr, ref.size()), ref, &worst), "replayed step differs from the oracle");
        }
        REQUIRE(engine.graph_ready(), "graph was not captured");
        REQUIRE(ops.contexts() == ctx_after_first, "a context was created after the first token (allocation inside capture)");
        // the cache planes are bit-identical to the oracle's mirror after all replays
        REQUIRE(download(T.at("kc").ptr, hk.size()) == hk, "K plane differs after replays");
        REQUIRE(download(T.at("vc").ptr, hv.size()) == hv, "V plane differs after replays");
    }
    cudaStreamDestroy(stream);
    std::printf("PASS: CUDA-graph capture-once contract (%s)\n", fused ? "fused five-input op" : "update + attention");
}
static void test_graph_contract() { run_graph_contract(false); }
static void test_graph_contract_fused() { run_graph_contract(true); }

// ---------------------------------------------------------------------------
static bool throws_with(const std::function<void()>& fn, const char* fragment) {
    try {
        fn();
    } catch (const std::runtime_error& e) {
        return std::strstr(e.what(), fragment) != nullptr;
    }
    return false;
}

static void test_error_behaviour() {
    sh::Engine engine;
    hkv::Registration<ShimBind> ops(engine);
    auto& T = engine.tensors();
    T.allocate_and_register("q", {1, 1, 4, 64}, sh::DType::FP16);
    T.allocate_and_register("k", {1, 16, 2, 64}, sh::DType::FP16);
    T.allocate_and_register("v", {1, 16, 2, 64}, sh::DType::FP16);
    T.allocate_and_register("o", {1, 1, 4, 64}, sh::DType::FP16);
    T.allocate_and_register("k32", {1, 16, 2, 64}, sh::DType::FP32);
    sh::CommandBuffer missing;
    missing.add_attention_cached("o", "q", "nope", "v", 4, 2, 64, 4, 16);
    REQUIRE(throws_with([&] { engine.execute(missing); }, "ATTENTION_CACHED: missing tensors"), "missing tensor must throw");
    sh::CommandBuffer dtype;
    dtype.add_attention_cached("o", "q", "k32", "v", 4, 2, 64, 4, 16);
    REQUIRE(throws_with([&] { engine.execute(dtype); }, "Expected FP16 tensor but got fp32"), "non-FP16 tensor must throw");
    sh::CommandBuffer geom;
    geom.add_attention_cached("o", "q", "k", "v", 4, 3, 64, 4, 16);
    REQUIRE(throws_with([&] { engine.execute(geom); }, "unsupported head geometry"), "H % KVH != 0 must throw");
    sh::CommandBuffer upd;
    upd.add_kv_cache_update("k", "v", "q", "nope", 0, 16, 2, 64, 1);
    REQUIRE(throws_with([&] { engine.execute(upd); }, "KV_CACHE_UPDATE: missing tensors"), "missing tensor must throw");
    // KV_CACHE_UPDATE with a batch and the engine's device position: the reference forwards the batch with
    // its ONE scalar (kernels/register_kernels.cpp:959-968) and every sequence writes at that position
    {
        const int B = 3, S = 16, KVH = 2, HD = 64, pos = 5;
        engine.alloc_device_cache_pos();
        T.allocate_and_register("bk_new", {(uint32_t)B, 1, (uint32_t)(KVH * HD)}, sh::DType::FP16);
        T.allocate_and_register("bv_new", {(uint32_t)B, 1, (uint32_t)(KVH * HD)}, sh::DType::FP16);
        T.allocate_and_register("bkc", {(uint32_t)B, (uint32_t)S, (uint32_t)KVH, (uint32_t)HD}, sh::DType::FP16);
        T.allocate_and_register("bvc", {(uint32_t)B, (uint32_t)S, (uint32_t)KVH, (uint32_t)HD}, sh::DType::FP16);
        std::vector<uint16_t> nk((size_t)B * KVH * HD), nv(nk.size()), hk((size_t)B * S * KVH * HD, 0), hv(hk.size(), 0);
        hkv_oracle_fill(nk.data(), 11, 0, nk.size());
        hkv_oracle_fill(nv.data(), 12, 0, nv.size());
        upload(T.at("bk_new").ptr, nk);
        upload(T.at("bv_new").ptr, nv);
        sh::CommandBuffer bupd;
        bupd.add_kv_cache_update("bkc", "bvc", "bk_new", "bv_new", 0, S, KVH, HD, 1);
        bupd.commands().back().set("device_pos", uint32_t{1});
        engine.update_device_cache_pos(pos, 1);
        engine.execute(bupd);
        cudaDeviceSynchronize();
        const int32_t same_pos[3] = {pos, pos, pos};
        hkv_oracle_append(nk.data(), nv.data(), hk.data(), hv.data(), B, 1, KVH, HD, S, (int64_t)S * KVH * HD, same_pos, 0);
        REQUIRE(download(T.at("bkc").ptr, hk.size()) == hk && download(T.at("bvc").ptr, hv.size()) == hv,
                "batched KV_CACHE_UPDATE writes every sequence at the engine's scalar position");
    }
    // a uint32 parameter stored as int32 is ignored (default used), as in the engine
    sh::Command c;
    c.set("head_dim", int32_t{64});
    REQUIRE(c.get<uint32_t>("head_dim", 128) == 128, "typed parameter lookup must be exact");
    REQUIRE(cudaGetLastError() == cudaSuccess, "no sticky CUDA error may remain");
    std::printf("PASS: error behaviour (missing tensors, dtype, geometry, typed params)\n");
}

// QK_NORM_ROPE in its fused seven-input form (writes the cache), device position.
static void test_qk_norm_rope_op() {
    const int H = 8, KVH = 2, HD = 128, S = 256, pos = 37;
    sh::Engine engine;
    hkv::Registration<ShimBind> ops(engine);
    engine.alloc_device_cache_pos();
    auto& T = engine.tensors();
    T.allocate_and_register("q", {1, 1, (uint32_t)(H * HD)}, sh::DType::FP16);
    T.allocate_and_register("k", {1, 1, (uint32_t)(KVH * HD)}, sh::DType::FP16);
    T.allocate_and_register("v", {1, 1, (uint32_t)(KVH * HD)}, sh::DType::FP16);
    T.allocate_and_register("qw", {(uint32_t)HD}, sh::DType::FP16);
    T.allocate_and_register("kw", {(uint32_t)HD}, sh::DType::FP16);
    T.allocate_and_register("kc", {1, (uint32_t)S, (uint32_t)KVH, (uint32_t)HD}, sh::DType::FP16);
    T.allocate_and_register("vc", {1, (uint32_t)S, (uint32_t)KVH, (uint32_t)HD}, sh::DType::FP16);
    std::vector<uint16_t> q((size_t)H * HD), k((size_t)KVH * HD), v((size_t)KVH * HD), qw(HD), kw(HD);
    hkv_oracle_fill(q.data(), 1, 0, q.size());
    hkv_oracle_fill(k.data(), 2, 0, k.size());
    hkv_oracle_fill(v.data(), 3, 0, v.size());
    for (int i = 0; i < HD; ++i) { qw[i] = hkv_oracle_f2h(1.0f + 0.01f * i); kw[i] = hkv_oracle_f2h(1.5f - 0.005f * i); }
    upload(T.at("q").ptr, q); upload(T.at("k").ptr, k); upload(T.at("v").ptr, v);
    upload(T.at("qw").ptr, qw); upload(T.at("kw").ptr, kw);
    sh::CommandBuffer cb;
    cb.add_op(sh::op::QK_NORM_ROPE(), "q")
        .in({"q", "k", "qw", "kw", "v", "kc", "vc"})
        .set("num_heads", uint32_t(H)).set("num_kv_heads", uint32_t(KVH)).set("dim", uint32_t(HD))
        .set("seq_len", uint32_t{1}).set("theta", 1000000.0f).set("max_seq_len", uint32_t(S))
        .set("device_pos", uint32_t{1});
    engine.update_device_cache_pos(pos, 1);
    engine.execute(cb);
    engine.sync();
    std::vector<uint16_t> rq = q, rk = k, rkc((size_t)S * KVH * HD, 0), rvc((size_t)S * KVH * HD, 0);
    const int32_t p32 = pos;
    hkv_oracle_qk_norm_rope(rq.data(), rk.data(), v.data(), qw.data(), kw.data(), rkc.data(), rvc.data(), 1, 1, H, KVH,
                            HD, HD, &p32, S, 0, 1e-6f, 1000000.0f, 1.0f);
    float worst;
    REQUIRE(close_enough(download(T.at("q").ptr, q.size()), rq, &worst), "rotated q differs from the oracle");
    REQUIRE(close_enough(download(T.at("kc").ptr, rkc.size()), rkc, &worst), "cache K differs from the oracle");
    REQUIRE(download(T.at("vc").ptr, rvc.size()) == rvc, "cache V must be bit-exact");
    REQUIRE(download(T.at("k").ptr, k.size()) == k, "k must stay untouched in the fused form");
    std::printf("PASS: QK_NORM_ROPE fused op (norm + rope + cache write)\n");
}

static void test_cache_owner() {
    hkv::KVCache cache;
    REQUIRE(!cache.allocate(hkv::KVCacheConfig{}), "zero dims refused");
    hkv::KVCacheConfig cfg;
    cfg.num_layers = 3; cfg.num_kv_heads = 2; cfg.head_dim = 64; cfg.max_batch_size = 2; cfg.max_seq_len = 32;
    REQUIRE(cache.allocate(cfg), "allocate");
    REQUIRE(cfg.total_bytes() == 3ull * 2 * 2 * 32 * 2 * 64 * 2, "byte budget");
    REQUIRE(cache.k_cache(3) == nullptr && cache.k_cache(2) == cache.k_cache(0) + 2 * (2 * 32 * 2 * 64), "layer stride");
    auto z = download(cache.v_cache(1), 2 * 32 * 2 * 64);
    for (uint16_t h : z) REQUIRE(h == 0, "planes are zero-filled");
    cache.advance(30); cache.advance(30);
    REQUIRE(cache.position() == 32, "advance clamps");
    cache.rewind_to(40);
    REQUIRE(cache.position() == 32, "rewind_to only moves back");
    cache.rewind_to(5);
    REQUIRE(cache.position() == 5, "rewind_to");
    const int32_t pos[2] = {7, 19};
    cache.set_positions(pos, nullptr);
    int32_t back[4];
    cudaMemcpy(back, cache.d_cache_pos(), sizeof back, cudaMemcpyDeviceToHost);
    REQUIRE(back[0] == 7 && back[1] == 19 && back[2] == 8 && back[3] == 20, "device positions");
    std::printf("PASS: C++ cache owner\n");
}

// ---------------------------------------------------------------------------
// Batched decode loop: sessions join and leave batch slots between tokens while ONE captured
// graph keeps replaying; every active slot must match its own batch-1 oracle history, a free slot
// must produce zeros and leave its planes untouched.
static void test_decode_loop() {
    const uint32_t L = 3, B = 4, H = 8, KVH = 2, HD = 64, S = 256;
    cudaStream_t stream;
    cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
    {
        hkv::DecodeLoopConfig cfg;
        cfg.layers = L; cfg.batch = B; cfg.heads = H; cfg.kv_heads = KVH; cfg.head_dim = HD; cfg.max_seq_len = S;
        hkv::BatchedDecodeLoop loop(cfg, stream);
        const size_t qn = (size_t)B * H * HD, kn = (size_t)B * KVH * HD, row = (size_t)KVH * HD;
        const size_t plane = (size_t)B * S * row;   // one layer
        half *d_q, *d_k, *d_v, *d_out;
        cudaMalloc(&d_q, L * qn * 2); cudaMalloc(&d_k, L * kn * 2); cudaMalloc(&d_v, L * kn * 2); cudaMalloc(&d_out, L * qn * 2);
        int hook_calls = 0;
        loop.bind(d_q, d_k, d_v, d_out, [&](uint32_t, cudaStream_t) { ++hook_calls; });

        // host mirror of the planes, [layer][slot][S][row]
        std::vector<uint16_t> hk(L * plane, 0), hv(L * plane, 0);
        int32_t mirror_pos[B];
        for (auto& p : mirror_pos) p = -1;
        auto attach = [&](uint32_t start) {
            const int slot = loop.board().attach(start);
            if (slot < 0) return slot;
            mirror_pos[slot] = (int32_t)start;
            // a new tenant starts from a prefix of `start` rows (zero rows here: only what it appends counts)
            return slot;
        };
        REQUIRE(attach(0) == 0, "first session takes slot 0");
        const float scale = 1.0f / std::sqrt(float(HD));
        const int steps = 40;
        int replays = 0;
        for (int s = 0; s < steps; ++s) {
            if (s == 3) REQUIRE(attach(0) == 1, "second session takes slot 1");
            if (s == 5) { REQUIRE(attach(0) == 2, "slot 2"); REQUIRE(attach(0) == 3, "slot 3"); REQUIRE(attach(0) == -1, "batch full"); }
            if (s == 12) { loop.board().detach(1); mirror_pos[1] = -1; }
            if (s == 20) {
                // slot 1 is re-let: the new tenant starts at row 0 and overwrites the old rows as it goes;
                // rows beyond its position are never attended
                REQUIRE(attach(0) == 1, "freed slot is reused");
            }
            if (s == 30) { loop.board().detach(0); mirror_pos[0] = -1; loop.board().detach(3); mirror_pos[3] = -1; }
            std::vector<uint16_t> q(L * qn), nk(L * kn), nv(L * kn);
            hkv_oracle_fill(q.data(), 1000 + s, 0, q.size());
            hkv_oracle_fill(nk.data(), 2000 + s, 0, nk.size());
            hkv_oracle_fill(nv.data(), 3000 + s, 0, nv.size());
            upload(d_q, q, stream); upload(d_k, nk, stream); upload(d_v, nv, stream);
            replays += loop.step() ? 1 : 0;
            cudaStreamSynchronize(stream);
            const auto out = download(d_out, L * qn);
            for (uint32_t l = 0; l < L; ++l)
                for (uint32_t b = 0; b < B; ++b) {
                    const uint16_t* o = out.data() + l * qn + (size_t)b * H * HD;
                    if (mirror_pos[b] < 0) {
                        for (size_t i = 0; i < (size_t)H * HD; ++i) REQUIRE(o[i] == 0, "free slot output is not zero");
                        continue;
                    }
                    uint16_t* pk = hk.data() + l * plane + (size_t)b * S * row;
                    uint16_t* pv = hv.data() + l * plane + (size_t)b * S * row;
                    const int32_t p = mirror_pos[b], tot = p + 1;
                    hkv_oracle_append(nk.data() + l * kn + b * row, nv.data() + l * kn + b * row, pk, pv, 1, 1, KVH, HD,
                                      S, 0, &p, 0);
                    std::vector<uint16_t> ref((size_t)H * HD), got(o, o + (size_t)H * HD);
                    hkv_oracle_decode(q.data() + l * qn + (size_t)b * H * HD, pk, pv, ref.data(), nullptr, 1, &tot, H,
                                      KVH, HD, S, 0, scale, 0, 0, 0, 1);
                    float worst;
                    REQUIRE(close_enough(got, ref, &worst), "slot output differs from its batch-1 oracle history");
                }
            for (auto& p : mirror_pos) if (p >= 0 && p < (int32_t)S) ++p;
            for (uint32_t b = 0; b < B; ++b)
                REQUIRE((mirror_pos[b] < 0 && !loop.board().active((int)b)) ||
                        (uint32_t)mirror_pos[b] == loop.board().position((int)b), "board position");
        }
        REQUIRE(loop.graph().valid(), "graph was not captured");
        REQUIRE(replays == steps, "every step, the first included, replays the captured graph");
        REQUIRE(loop.graph().capture_failures() == 0, "capture failed");
        REQUIRE(hook_calls == (int)L, "the per-layer hook runs at capture only");
        REQUIRE(loop.device_status() == 0, "device status word");
        // planes: bit-identical to the mirror (free slots included: nothing was written for them)
        for (uint32_t l = 0; l < L; ++l) {
            REQUIRE(download(loop.cache().k_cache(l), plane) == std::vector<uint16_t>(hk.begin() + l * plane, hk.begin() + (l + 1) * plane), "K plane differs");
            REQUIRE(download(loop.cache().v_cache(l), plane) == std::vector<uint16_t>(hv.begin() + l * plane, hv.begin() + (l + 1) * plane), "V plane differs");
        }
        // capture failure → per-token fallback, sticky error cleared
        hkv::GraphReplay g2(1);
        int direct = 0;
        const bool r = g2.run(stream, [&](cudaStream_t st) {
            ++direct;
            if (direct == 1) cudaStreamSynchronize(st);   // illegal during capture: invalidates it
        });
        REQUIRE(!r && direct == 2 && g2.capture_failures() == 1 && !g2.valid(), "failed capture falls back to direct enqueue");
        REQUIRE(cudaGetLastError() == cudaSuccess, "sticky error left behind");
        REQUIRE(!g2.run(stream, [&](cudaStream_t) { ++direct; }) && direct == 3, "gives up capturing after the limit");
        cudaFree(d_q); cudaFree(d_k); cudaFree(d_v); cudaFree(d_out);
    }
    cudaStreamDestroy(stream);
    std::printf("PASS: batched decode loop (sessions join/leave under one captured graph)\n");
}

int main(int argc, char** argv) {
    struct Case { const char* name; void (*fn)(); };
    const Case cases[] = {{"known_answers", test_known_answers}, {"graph_contract", test_graph_contract},
                          {"graph_contract_fused", test_graph_contract_fused},
                          {"error_behaviour", test_error_behaviour}, {"qk_norm_rope_op", test_qk_norm_rope_op},
                          {"cache_owner", test_cache_owner}, {"decode_loop", test_decode_loop}};
    if (argc > 1 && std::strcmp(argv[1], "--list") == 0) {
        for (const auto& c : cases) std::printf("%s\n", c.name);
        return 0;
    }
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        std::printf("FAIL: no CUDA device\n");
        return 2;
    }
    for (const auto& c : cases) c.fn();
    std::printf("%s (%d failure(s))\n", g_failures ? "FAILED" : "ALL PASSED", g_failures);
    return g_failures ? 1 : 0;
}
