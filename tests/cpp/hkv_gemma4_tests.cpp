// hkv_gemma4_tests.cpp — C++ tests of the heterogeneous / shared KV cache owner
// (host/hkv_gemma4_kv_cache.hpp) and of the per-layer decode loop (host/hkv_decode_loop.hpp) on a B200.
//
//   layout_and_aliases   the reference's own known answers for the layout (reference
//                        tests/test_gemma4_kv.cu:110-153): 35 synthetic layers, every fifth global
//                        (head_dim 512) the others local (head_dim 256, window 512), 20 shared:
//                        15 physical slots, layers 15-18 alias layer 13, 19-34 alias layer 14, true
//                        pointer aliases, 147 456 bytes for 8 positions, tensor names and shapes.
//   layer_plan           what the reference's graph emission fixes per layer
//                        (tests/test_gemma4_kv.cu:155-228, src/graph_builder.cpp:699, :746, :767-777):
//                        owners append (15 of 35), shared layers only attend their owner's plane,
//                        local layers carry window 512, global ones none, scale 1.0 everywhere.
//   decode_local_global_shared
//                        12 layers, five local (ring planes) per global one, the last four shared,
//                        three sessions at different positions (one crossing the ring's wrap), 14
//                        tokens under ONE captured graph: every layer's output of every token equals
//                        the oracle's linear-plane + window-mask result, owner planes end bit-exact,
//                        and the K/V rows offered to shared layers (poisoned with NaN) never land.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "hkv.h"
#include "hkv_decode_loop.hpp"
#include "hkv_gemma4_kv_cache.hpp"

extern "C" {
void hkv_oracle_fill(uint16_t* dst, uint64_t seed, uint64_t first_index, uint64_t count);
void hkv_oracle_append(const uint16_t* new_k, const uint16_t* new_v, uint16_t* k_cache, uint16_t* v_cache,
                       int B, int S, int KVH, int HD, int slots, int64_t batch_stride, const int32_t* pos,
                       int layout);
void hkv_oracle_decode(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out,
                       float* out_f32, int B, const int32_t* total, int H, int KVH, int HD, int slots,
                       int64_t batch_stride, float scale, int window, int layout, int mode, int threads);
float hkv_oracle_h2f(uint16_t h);
}

static int g_failures = 0;
#define REQUIRE(cond, msg)                                              \
    do {                                                                \
        if (!(cond)) {                                                  \
            std::printf("FAIL: %s (%s:%d)\n", msg, __FILE__, __LINE__); \
            ++g_failures;                                               \
        }                                                               \
    } while (0)

namespace {

std::vector<hkv::Gemma4LayerSpec> synthetic_gemma(uint32_t layers) {
    std::vector<hkv::Gemma4LayerSpec> out(layers);
    for (uint32_t i = 0; i < layers; ++i) {
        out[i].is_global = i % 5 == 4;
        out[i].sliding_window = out[i].is_global ? 0 : 512;
        out[i].head_dim = out[i].is_global ? 512 : 256;
    }
    return out;
}

void test_layout_and_aliases() {
    hkv::Gemma4KVCache cache;
    REQUIRE(cache.allocate(synthetic_gemma(35), 20, 1, 1, 8), "allocate heterogeneous KV cache");
    REQUIRE(cache.num_layers() == 35 && cache.physical_slots() == 15, "only the first 15 layers own physical KV slots");
    REQUIRE(cache.source_layer(13) == 13 && cache.source_layer(14) == 14, "source layers own their slots");
    REQUIRE(cache.source_layer(15) == 13 && cache.source_layer(18) == 13, "shared local layers reuse layer 13");
    REQUIRE(cache.source_layer(19) == 14 && cache.source_layer(34) == 14, "shared global layers reuse layer 14");
    REQUIRE(cache.k_cache(15) == cache.k_cache(13) && cache.v_cache(19) == cache.v_cache(14), "shared layers are true pointer aliases");
    REQUIRE(cache.head_dim(13) == 256 && cache.head_dim(14) == 512, "local/global slot dimensions remain heterogeneous");
    REQUIRE(cache.total_bytes() == 147456, "heterogeneous KV byte budget for 8 positions");
    REQUIRE(cache.is_shared(15) && !cache.is_shared(14) && cache.source_layer(35) == 0xFFFFFFFFu, "is_shared / out-of-range layer");

    const half value = __float2half(7.0f);
    REQUIRE(cudaMemcpy(cache.k_cache(13), &value, sizeof value, cudaMemcpyHostToDevice) == cudaSuccess, "write local source alias");
    half observed{};
    REQUIRE(cudaMemcpy(&observed, cache.k_cache(15), sizeof observed, cudaMemcpyDeviceToHost) == cudaSuccess, "read shared local alias");
    REQUIRE(__half2float(observed) == 7.0f, "shared alias observes source writes");

    struct Entry { void* ptr; std::vector<uint32_t> shape; };
    std::map<std::string, Entry> registry;
    cache.register_tensors([&](const std::string& name, half* ptr, const std::vector<uint32_t>& shape) { registry[name] = Entry{ptr, shape}; },
                           "_g4kv");
    REQUIRE(registry.size() == 70, "k and v of all 35 layers are published");
    REQUIRE((registry["_g4kv.layer13.k"].shape == std::vector<uint32_t>{1, 8, 1, 256}), "local cache tensor shape");
    REQUIRE((registry["_g4kv.layer14.k"].shape == std::vector<uint32_t>{1, 8, 1, 512}), "global cache tensor shape");
    REQUIRE(registry["_g4kv.layer15.k"].ptr == registry["_g4kv.layer13.k"].ptr, "registered local tensor is an alias");

    // position bookkeeping, as KVCache (src/gemma4_kv_cache.hpp:179-187)
    cache.advance(5); cache.advance(9);
    REQUIRE(cache.position() == 8, "advance clamps to max_seq_len");
    cache.rewind_to(3); cache.rewind_to(6);
    REQUIRE(cache.position() == 3, "rewind_to only moves backwards");

    // where the reference's allocate() returns false
    hkv::Gemma4KVCache bad;
    REQUIRE(!bad.allocate({}, 0, 1, 1, 8), "no layers");
    REQUIRE(!bad.allocate(synthetic_gemma(35), 36, 1, 1, 8), "more shared layers than layers");
    REQUIRE(!bad.allocate(synthetic_gemma(35), 35, 1, 1, 8), "no owner at all");
    REQUIRE(!bad.allocate(synthetic_gemma(35), 31, 1, 1, 8), "a shared global layer without a global owner (owners 0..3 are local)");
    auto mism = synthetic_gemma(35);
    mism[20].head_dim = 128;
    REQUIRE(!bad.allocate(mism, 20, 1, 1, 8) && !bad.is_allocated(), "a shared layer whose head_dim differs from its owner's");

    // ring planes for local owners (not in the reference): 8 local owners shrink to 4 rows each
    hkv::Gemma4KVCache ring;
    REQUIRE(ring.allocate(synthetic_gemma(35), 20, 1, 1, 8, 4), "allocate with ring planes");
    REQUIRE(ring.rows(13) == 4 && ring.is_ring(13) && ring.rows(15) == 4 && ring.rows(14) == 8 && !ring.is_ring(14), "local owners and their aliases are rings");
    REQUIRE(ring.total_bytes() == 2 * 2 * (size_t)(12 * 4 * 256 + 3 * 8 * 512), "ring byte budget");
}

void test_layer_plan() {
    hkv::Gemma4KVCache cache;
    REQUIRE(cache.allocate(synthetic_gemma(35), 20, 1, 1, 8), "allocate");
    const std::vector<hkv::DecodeLayer> plan = hkv::decode_layers_of(cache, 1.0f);
    size_t appends = 0;
    for (const hkv::DecodeLayer& d : plan) appends += d.append;
    REQUIRE(plan.size() == 35 && appends == 15, "complete forward updates only the 15 physical source layers");
    REQUIRE(plan[13].append && plan[13].head_dim == 256 && plan[13].window == 512 && plan[13].scale == 1.0f,
            "local cached attention geometry, window and scale");
    REQUIRE(!plan[15].append && plan[15].k_plane == cache.k_cache(13) && plan[15].window == 512, "shared local layer consumes the layer-13 alias and writes nothing");
    REQUIRE(!plan[19].append && plan[19].head_dim == 512 && plan[19].window == 0 && plan[19].k_plane == cache.k_cache(14) && plan[19].scale == 1.0f,
            "shared global layer uses full HD512 attention over layer 14's KV without updating it");
}

bool close_enough(const uint16_t* got, const uint16_t* ref, size_t n, float* worst) {
    bool ok = true;
    for (size_t i = 0; i < n; ++i) {
        const float g = hkv_oracle_h2f(got[i]), r = hkv_oracle_h2f(ref[i]);
        const float err = std::fabs(g - r);
        if (!(err <= 2e-3f + 1e-2f * std::fabs(r))) ok = false;   // the path's tolerance (NaN fails too)
        else if (err > *worst) *worst = err;
    }
    return ok;
}

void test_decode_local_global_shared() {
    // 12 layers: l % 6 == 5 global (head_dim 512, linear plane), the rest local (head_dim 256, window =
    // ring of 128 rows). The last 4 layers are shared: 8, 9, 10 (local) -> layer 7, 11 (global) -> layer 5.
    constexpr uint32_t NL = 12, B = 3, H = 8, KVH = 2, MAXSEQ = 512, W = 128, STEPS = 14;
    std::vector<hkv::Gemma4LayerSpec> specs(NL);
    for (uint32_t l = 0; l < NL; ++l) {
        specs[l].is_global = l % 6 == 5;
        specs[l].head_dim = specs[l].is_global ? 512 : 256;
        specs[l].sliding_window = specs[l].is_global ? 0 : W;
    }
    hkv::Gemma4KVCache cache;
    REQUIRE(cache.allocate(specs, 4, KVH, B, MAXSEQ, W), "allocate the 12-layer cache with ring planes");
    REQUIRE(cache.source_layer(8) == 7 && cache.source_layer(10) == 7 && cache.source_layer(11) == 5, "aliases");
    cudaStream_t stream;
    REQUIRE(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess, "stream");
    try {
        hkv::BatchedDecodeLoop loop(B, H, KVH, MAXSEQ, hkv::decode_layers_of(cache, 1.0f / 16.0f), stream);
        REQUIRE(loop.contexts() == 2, "one context per distinct layer geometry (local ring, global linear)");
        const size_t QN = loop.q_elems(), KN = loop.kv_elems();
        half *dq, *dkn, *dvn, *dout;
        cudaMalloc(&dq, QN * 2); cudaMalloc(&dkn, KN * 2); cudaMalloc(&dvn, KN * 2); cudaMalloc(&dout, QN * 2);
        loop.bind(dq, dkn, dvn, dout);
        // three sessions: deep into the ring, at the start, just before the ring's first wrap
        const uint32_t start[B] = {300, 5, 120};
        // host mirror: LINEAR planes of MAXSEQ rows per owner layer (the reference's layout), pre-filled
        // below each session's start; the device planes get the same rows (ring: the last W of them)
        std::vector<std::vector<uint16_t>> mk(NL), mv(NL);
        for (uint32_t l = 0; l < NL; ++l) {
            if (cache.is_shared(l)) continue;
            const uint32_t HD = specs[l].head_dim, row = KVH * HD, rows = cache.rows(l);
            mk[l].assign((size_t)B * MAXSEQ * row, 0); mv[l].assign((size_t)B * MAXSEQ * row, 0);
            std::vector<uint16_t> dk((size_t)B * rows * row, 0), dv((size_t)B * rows * row, 0);
            for (uint32_t b = 0; b < B; ++b) {
                hkv_oracle_fill(&mk[l][(size_t)b * MAXSEQ * row], 0x6100 + l * 16 + b, 0, (size_t)start[b] * row);
                hkv_oracle_fill(&mv[l][(size_t)b * MAXSEQ * row], 0x6200 + l * 16 + b, 0, (size_t)start[b] * row);
                for (uint32_t p = 0; p < start[b]; ++p) {
                    const uint32_t r = cache.is_ring(l) ? p % rows : p;
                    std::memcpy(&dk[((size_t)b * rows + r) * row], &mk[l][((size_t)b * MAXSEQ + p) * row], row * 2);
                    std::memcpy(&dv[((size_t)b * rows + r) * row], &mv[l][((size_t)b * MAXSEQ + p) * row], row * 2);
                }
            }
            cudaMemcpy(cache.k_cache(l), dk.data(), dk.size() * 2, cudaMemcpyHostToDevice);
            cudaMemcpy(cache.v_cache(l), dv.data(), dv.size() * 2, cudaMemcpyHostToDevice);
        }
        int slot[B];
        for (uint32_t b = 0; b < B; ++b) slot[b] = loop.board().attach(start[b]);
        REQUIRE(slot[0] == 0 && slot[1] == 1 && slot[2] == 2, "sessions take the batch slots in order");

        std::vector<uint16_t> q(QN), nk(KN), nv(KN), got(QN), ref;
        float worst = 0.0f;
        uint64_t replays = 0;
        bool all_ok = true;
        for (uint32_t s = 0; s < STEPS; ++s) {
            hkv_oracle_fill(q.data(), 0x8100 + s, 0, QN);
            hkv_oracle_fill(nk.data(), 0x8200 + s, 0, KN);
            hkv_oracle_fill(nv.data(), 0x8300 + s, 0, KN);
            for (uint32_t l = 0; l < NL; ++l)   // what a shared layer is offered must never be read or stored
                if (cache.is_shared(l))
                    for (size_t i = loop.kv_offset(l); i < loop.kv_offset(l + 1); ++i) nk[i] = nv[i] = 0x7E00;   // NaN
            cudaMemcpyAsync(dq, q.data(), QN * 2, cudaMemcpyHostToDevice, stream);
            cudaMemcpyAsync(dkn, nk.data(), KN * 2, cudaMemcpyHostToDevice, stream);
            cudaMemcpyAsync(dvn, nv.data(), KN * 2, cudaMemcpyHostToDevice, stream);
            int32_t pos[B], total[B];
            for (uint32_t b = 0; b < B; ++b) { pos[b] = (int32_t)loop.board().position(slot[b]); total[b] = pos[b] + 1; }
            replays += loop.step() ? 1 : 0;
            cudaStreamSynchronize(stream);
            cudaMemcpy(got.data(), dout, QN * 2, cudaMemcpyDeviceToHost);
            for (uint32_t l = 0; l < NL; ++l) {
                const uint32_t HD = specs[l].head_dim, row = KVH * HD, src = cache.source_layer(l);
                if (!cache.is_shared(l))
                    hkv_oracle_append(&nk[loop.kv_offset(l)], &nv[loop.kv_offset(l)], mk[l].data(), mv[l].data(), B, 1, KVH, HD, MAXSEQ,
                                      (int64_t)MAXSEQ * row, pos, 0);
                ref.assign((size_t)B * H * HD, 0);
                hkv_oracle_decode(&q[loop.q_offset(l)], mk[src].data(), mv[src].data(), ref.data(), nullptr, B, total, H, KVH, HD, MAXSEQ,
                                  (int64_t)MAXSEQ * row, 1.0f / 16.0f, specs[l].is_global ? 0 : (int)W, 0, 0, 4);
                if (!close_enough(&got[loop.q_offset(l)], ref.data(), ref.size(), &worst)) {
                    all_ok = false;
                    std::printf("  mismatch: token %u layer %u\n", s, l);
                }
            }
        }
        REQUIRE(all_ok, "every layer of every token equals the oracle's linear + window-mask result");
        REQUIRE(replays == STEPS, "every step replays the one captured graph");
        REQUIRE(loop.graph().node_count() >= NL * 2, "all layers sit in that graph");
        REQUIRE(loop.device_status() == 0, "device status words clean");
        // owner planes: bit-exact images of the mirror (ring: the last W positions at position mod W)
        bool planes_ok = true;
        for (uint32_t l = 0; l < NL && planes_ok; ++l) {
            if (cache.is_shared(l)) continue;
            const uint32_t HD = specs[l].head_dim, row = KVH * HD, rows = cache.rows(l);
            std::vector<uint16_t> dk((size_t)B * rows * row), dv(dk.size());
            cudaMemcpy(dk.data(), cache.k_cache(l), dk.size() * 2, cudaMemcpyDeviceToHost);
            cudaMemcpy(dv.data(), cache.v_cache(l), dv.size() * 2, cudaMemcpyDeviceToHost);
            for (uint32_t b = 0; b < B && planes_ok; ++b) {
                const uint32_t end = start[b] + STEPS, first = cache.is_ring(l) && end > rows ? end - rows : 0;
                for (uint32_t p = first; p < end; ++p) {
                    const uint32_t r = cache.is_ring(l) ? p % rows : p;
                    if (std::memcmp(&dk[((size_t)b * rows + r) * row], &mk[l][((size_t)b * MAXSEQ + p) * row], row * 2) ||
                        std::memcmp(&dv[((size_t)b * rows + r) * row], &mv[l][((size_t)b * MAXSEQ + p) * row], row * 2)) {
                        planes_ok = false;
                        std::printf("  plane mismatch: layer %u seq %u position %u\n", l, b, p);
                        break;
                    }
                }
            }
        }
        REQUIRE(planes_ok, "owner planes bit-exact; nothing offered to a shared layer was stored");
        std::printf("  %u tokens x %u layers, %llu replays, %zu graph nodes, max abs err %.3e\n", STEPS, NL,
                    (unsigned long long)replays, loop.graph().node_count(), worst);
        cudaFree(dq); cudaFree(dkn); cudaFree(dvn); cudaFree(dout);
    } catch (const std::exception& e) {
        std::printf("FAIL: exception: %s\n", e.what());
        ++g_failures;
    }
    cudaStreamDestroy(stream);
}

}  // namespace

int main(int argc, char** argv) {
    struct Case { const char* name; void (*fn)(); };
    const Case cases[] = {{"layout_and_aliases", test_layout_and_aliases},
                          {"layer_plan", test_layer_plan},
                          {"decode_local_global_shared", test_decode_local_global_shared}};
    if (argc > 1 && std::string(argv[1]) == "--list") {
        for (const Case& c : cases) std::printf("%s\n", c.name);
        return 0;
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("FAIL: no CUDA device\n"); return 1; }
    for (const Case& c : cases) {
        const int before = g_failures;
        c.fn();
        std::printf("%s: %s\n", g_failures == before ? "PASS" : "FAIL", c.name);
    }
    if (g_failures == 0) std::printf("ALL PASSED\n");
    return g_failures ? 1 : 0;
}
