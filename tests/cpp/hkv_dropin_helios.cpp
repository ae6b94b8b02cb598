// hkv_dropin_helios.cpp — drop-in test at the REAL engine's registry boundary.
//
// This translation unit is compiled against the reference engine's own headers and linked
// with the reference's own engine core and kernels (compiled from the reference checkout
// where it lies; recipe: `make -C oracle dropin`, output oracle/_ref/hkv_dropin_helios).
// It registers all reference kernels, then installs libhkv's ops over them with
// hkv::Registration<HeliosBind>, and drives the engine exactly as its sessions do:
//   * the known-answer command buffers of the reference's hot-path test
//     (reference tests/test_gemma4_kv.cu:234-347), first through the reference kernels,
//     then through libhkv — both must give the known answers;
//   * the capture-once CUDA-graph decode loop (reference src/inference_session.cpp:248-276,
//     src/engine.cpp:151-269): first token execute(), later tokens execute_graph_replay(),
//     update_device_cache_pos() before each; every token checked against the CPU oracle and
//     against the reference kernels run on a copy of the same cache.
// Test infrastructure only; needs a GPU.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "engine.hpp"   // reference src/
#include "kernels.hpp"  // reference kernels/
#include "hkv.h"
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
}

struct HeliosBind {
    using Engine = helios::Engine;
    using ExecContext = helios::ExecContext;
    using Command = helios::Command;
    using TensorInfo = helios::TensorInfo;
    static uint32_t attention_cached() { return helios::op::ATTENTION_CACHED(); }
    static uint32_t kv_cache_update() { return helios::op::KV_CACHE_UPDATE(); }
    static uint32_t attention_prefill_cached() { return helios::op::ATTENTION_PREFILL_CACHED(); }
    static uint32_t qk_norm_rope() { return helios::op::QK_NORM_ROPE(); }
    static bool is_fp16(const TensorInfo& t) { return t.dtype == helios::dtype::FP16(); }
    static const char* dtype_name(const TensorInfo& t) { return helios::dtype_name(t.dtype); }
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

static void upload(void* dst, const std::vector<uint16_t>& src) {
    cudaMemcpy(dst, src.data(), src.size() * 2, cudaMemcpyHostToDevice);
}
static std::vector<uint16_t> download(const void* src, size_t n) {
    std::vector<uint16_t> out(n);
    cudaMemcpy(out.data(), src, n * 2, cudaMemcpyDeviceToHost);
    return out;
}
static bool close_enough(const std::vector<uint16_t>& got, const std::vector<uint16_t>& ref) {
    for (size_t i = 0; i < got.size(); ++i) {
        const float x = hkv_oracle_h2f(got[i]), r = hkv_oracle_h2f(ref[i]);
        if (!(std::fabs(x - r) <= 2e-3f + 1e-2f * std::fabs(r))) return false;
    }
    return true;
}
static helios::EngineConfig config_on(cudaStream_t s) {
    helios::EngineConfig cfg;
    cfg.scratch_pool.auto_fraction = 0.0f;
    cfg.scratch_pool.min_size_bytes = 0;
    cfg.stream = s;
    return cfg;
}

// The reference test's known answers, with either the reference kernels or libhkv installed.
static void known_answers(bool use_hkv) {
    helios::Engine engine(config_on(nullptr));
    helios::kernels::register_all_kernels(engine);
    std::unique_ptr<hkv::Registration<HeliosBind>> ops;
    if (use_hkv) ops.reset(new hkv::Registration<HeliosBind>(engine));
    auto& T = engine.tensors();
    const auto F16 = helios::dtype::FP16();
    T.allocate_and_register("attn.q", {1, 1, 1, 2}, F16, true);
    T.allocate_and_register("attn.k", {1, 6, 1, 2}, F16, true);
    T.allocate_and_register("attn.v", {1, 6, 1, 2}, F16, true);
    T.allocate_and_register("attn.out", {1, 1, 1, 2}, F16, true);
    std::vector<uint16_t> v(12);
    for (int p = 0; p < 6; ++p) v[p * 2] = v[p * 2 + 1] = hkv_oracle_f2h(float(p + 1));
    upload(T.at("attn.v").ptr, v);
    helios::CommandBuffer local;
    local.add_attention_cached("attn.out", "attn.q", "attn.k", "attn.v", 1, 1, 2, 6, 6, 3);
    engine.execute(local);
    engine.sync();
    auto out = download(T.at("attn.out").ptr, 2);
    REQUIRE(std::fabs(hkv_oracle_h2f(out[0]) - 5.0f) < 0.01f, "decode local window: mean of 4,5,6");

    T.allocate_and_register("prefill.q", {1, 2, 1, 2}, F16, true);
    T.allocate_and_register("prefill.out", {1, 2, 1, 2}, F16, true);
    helios::CommandBuffer prefill;
    prefill.add_op(helios::op::ATTENTION_PREFILL_CACHED(), "prefill.out")
        .in({"prefill.q", "attn.k", "attn.v"})
        .set("num_heads", uint32_t{1}).set("num_kv_heads", uint32_t{1}).set("head_dim", uint32_t{2})
        .set("scale", 1.0f).set("seq_len", uint32_t{2}).set("past_len", uint32_t{4})
        .set("max_seq_len", uint32_t{6}).set("window_size", uint32_t{3});
    engine.execute(prefill);
    engine.sync();
    auto pout = download(T.at("prefill.out").ptr, 4);
    REQUIRE(std::fabs(hkv_oracle_h2f(pout[0]) - 4.0f) < 0.01f && std::fabs(hkv_oracle_h2f(pout[2]) - 5.0f) < 0.01f,
            "prefill window slides per query");

    T.allocate_and_register("boundary.k", {1, 514, 1, 2}, F16, true);
    T.allocate_and_register("boundary.v", {1, 514, 1, 2}, F16, true);
    T.allocate_and_register("boundary.out", {1, 1, 1, 2}, F16, true);
    std::vector<uint16_t> bv(514 * 2, hkv_oracle_f2h(2.0f));
    for (int i = 0; i < 4; ++i) bv[i] = hkv_oracle_f2h(1000.0f);
    upload(T.at("boundary.v").ptr, bv);
    helios::CommandBuffer boundary;
    boundary.add_attention_cached("boundary.out", "attn.q", "boundary.k", "boundary.v", 1, 1, 2, 514, 514, 512);
    engine.execute(boundary);
    engine.sync();
    REQUIRE(std::fabs(hkv_oracle_h2f(download(T.at("boundary.out").ptr, 2)[0]) - 2.0f) < 0.01f, ">512 window boundary");

    T.allocate_and_register("global.q", {1, 1, 1, 512}, F16, true);
    T.allocate_and_register("global.k", {1, 2, 1, 512}, F16, true);
    T.allocate_and_register("global.v", {1, 2, 1, 512}, F16, true);
    T.allocate_and_register("global.out", {1, 1, 1, 512}, F16, true);
    std::vector<uint16_t> gv(1024, hkv_oracle_f2h(2.0f));
    for (size_t i = 512; i < 1024; ++i) gv[i] = hkv_oracle_f2h(6.0f);
    upload(T.at("global.v").ptr, gv);
    helios::CommandBuffer global;
    global.add_attention_cached("global.out", "global.q", "global.k", "global.v", 1, 1, 512, 2, 2);
    engine.execute(global);
    engine.sync();
    for (uint16_t h : download(T.at("global.out").ptr, 512))
        REQUIRE(std::fabs(hkv_oracle_h2f(h) - 4.0f) < 0.01f, "HD512 writes every dimension");
    std::printf("PASS: known answers through helios::Engine with %s\n", use_hkv ? "libhkv ops" : "reference kernels");
}
static void test_known_answers_reference() { known_answers(false); }
static void test_known_answers_hkv() { known_answers(true); }

// The engine's decode loop with capture-once graph replay, libhkv vs reference kernels vs oracle.
static void test_graph_decode_loop() {
    const int H = 28, KVH = 4, HD = 128, S = 4096, start = 2000, steps = 16;
    const size_t row = (size_t)KVH * HD;
    const float scale = 1.0f / std::sqrt(float(HD));
    cudaStream_t s_hkv, s_ref;
    cudaStreamCreateWithFlags(&s_hkv, cudaStreamNonBlocking);
    cudaStreamCreateWithFlags(&s_ref, cudaStreamNonBlocking);
    {
        helios::Engine eng_hkv(config_on(s_hkv)), eng_ref(config_on(s_ref));
        helios::kernels::register_all_kernels(eng_hkv);
        helios::kernels::register_all_kernels(eng_ref);
        hkv::Registration<HeliosBind> ops(eng_hkv);  // overwrites the three attention ops
        std::vector<uint16_t> hk((size_t)S * row, 0), hv((size_t)S * row, 0);
        hkv_oracle_fill(hk.data(), 21, 0, (uint64_t)start * row);
        hkv_oracle_fill(hv.data(), 22, 0, (uint64_t)start * row);
        helios::Engine* engines[2] = {&eng_hkv, &eng_ref};
        const auto F16 = helios::dtype::FP16();
        for (auto* e : engines) {
            e->alloc_device_cache_pos();
            auto& T = e->tensors();
            T.allocate_and_register("q", {1, 1, (uint32_t)H, (uint32_t)HD}, F16, true);
            T.allocate_and_register("k_new", {1, 1, (uint32_t)row}, F16, true);
            T.allocate_and_register("v_new", {1, 1, (uint32_t)row}, F16, true);
            T.allocate_and_register("kc", {1, (uint32_t)S, (uint32_t)KVH, (uint32_t)HD}, F16, true);
            T.allocate_and_register("vc", {1, (uint32_t)S, (uint32_t)KVH, (uint32_t)HD}, F16, true);
            T.allocate_and_register("out", {1, 1, (uint32_t)H, (uint32_t)HD}, F16, true);
            upload(T.at("kc").ptr, hk);
            upload(T.at("vc").ptr, hv);
        }
        // what the graph builder emits for a cached decode layer (reference src/graph_builder.cpp:1340-1358)
        helios::CommandBuffer cb;
        cb.add_kv_cache_update("kc", "vc", "k_new", "v_new", 0, S, KVH, HD, 1);
        cb[cb.size() - 1].set("device_pos", uint32_t{1});
        cb.add_attention_cached("out", "q", "kc", "vc", H, KVH, HD, 1, S, 0);
        cb[cb.size() - 1].set("device_pos", uint32_t{1});

        for (int s = 0; s < steps; ++s) {
            const int pos = start + s;
            std::vector<uint16_t> q((size_t)H * HD), nk(row), nv(row);
            hkv_oracle_fill(q.data(), 100 + s, 0, q.size());
            hkv_oracle_fill(nk.data(), 200 + s, 0, row);
            hkv_oracle_fill(nv.data(), 300 + s, 0, row);
            for (auto* e : engines) {
                auto& T = e->tensors();
                upload(T.at("q").ptr, q);
                upload(T.at("k_new").ptr, nk);
                upload(T.at("v_new").ptr, nv);
                e->update_device_cache_pos(pos, 1);
                if (s == 0) e->execute(cb);
                else e->execute_graph_replay(cb);
                e->sync();
            }
            const int32_t p32 = pos, tot = pos + 1;
            hkv_oracle_append(nk.data(), nv.data(), hk.data(), hv.data(), 1, 1, KVH, HD, S, 0, &p32, 0);
            std::vector<uint16_t> ref((size_t)H * HD);
            hkv_oracle_decode(q.data(), hk.data(), hv.data(), ref.data(), nullptr, 1, &tot, H, KVH, HD, S, 0, scale, 0,
                              0, 0, 4);
            const auto got_hkv = download(eng_hkv.tensors().at("out").ptr, ref.size());
            const auto got_ref = download(eng_ref.tensors().at("out").ptr, ref.size());
            REQUIRE(close_enough(got_hkv, ref), "libhkv token differs from the oracle");
            REQUIRE(close_enough(got_ref, ref), "reference token differs from the oracle");
            REQUIRE(close_enough(got_hkv, got_ref), "libhkv token differs from the reference kernels");
        }
        REQUIRE(eng_hkv.graph_ready(), "the engine did not capture a graph with libhkv ops installed");
        REQUIRE(eng_ref.graph_ready(), "the engine did not capture a graph with its own ops");
        // both engines' cache planes are bit-identical to each other and to the oracle's mirror
        REQUIRE(download(eng_hkv.tensors().at("kc").ptr, hk.size()) == hk, "K plane (libhkv) differs from the oracle");
        REQUIRE(download(eng_ref.tensors().at("kc").ptr, hk.size()) == hk, "K plane (reference) differs from the oracle");
        REQUIRE(download(eng_hkv.tensors().at("vc").ptr, hv.size()) == hv, "V plane (libhkv) differs from the oracle");
    }
    cudaStreamDestroy(s_hkv);
    cudaStreamDestroy(s_ref);
    std::printf("PASS: capture-once decode loop through helios::Engine (libhkv == reference kernels == oracle)\n");
}

int main(int argc, char** argv) {
    struct Case { const char* name; void (*fn)(); };
    const Case cases[] = {{"known_answers_reference", test_known_answers_reference},
                          {"known_answers_hkv", test_known_answers_hkv},
                          {"graph_decode_loop", test_graph_decode_loop}};
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
