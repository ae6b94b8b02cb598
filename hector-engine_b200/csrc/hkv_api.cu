// hkv_api.cu — the C ABI of libhkv (declared in include/hkv.h): argument validation,
// context and workspace ownership, tensor-map encoding and kernel dispatch.
// Host side only enqueues work; there is no CPU compute path in this library.

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <map>
#include <utility>
#include <vector>

#include "../../include/hkv.h"
#include "hkv_basic.cuh"
#include "hkv_decode_tma.cuh"
#include "hkv_prefill.cuh"
#include "hkv_prefill_tc.cuh"
#include "hkv_prefill_tc2.cuh"
#include "hkv_rope.cuh"

using namespace hkv;

// ---------------------------------------------------------------------------
// Context
// ---------------------------------------------------------------------------
struct TmapPair {
    CUtensorMap k, v;
};

struct hkv_ctx {
    hkv_geometry g;
    SeqMap map;
    int device = -1;
    int sm_count = 0;
    size_t smem_optin = 0;
    int G = 0;
    long long batch_stride = 0;
    int chunk_tiles = 1, max_chunks = 1;
    int kernel = HKV_KERNEL_GENERIC;  // preferred kernel
    int tma_groups = 2;
    TmaSmemPlan plan{0, 0};
    float* workspace = nullptr;     // chunked split-K partials (any-geometry kernel)
    size_t workspace_bytes = 0;
    float* span_ws = nullptr;       // equal-span partials of the TMA kernel: [2*SMs + batch][H][HD+2]
    int* span_gpre = nullptr;       // [batch + 1] tile table the TMA kernel leaves for the merge
    int span_gang = 1;              // CTAs sharing a span (gcd of the kv heads and the grid)
    int tma_grid = 0;               // persistent grid of the TMA kernel
    int32_t* d_status = nullptr;
    long long q_stride = 0, new_stride = 0;   // elements between sequences' q / k_new rows in decode-side calls
    bool ready = false;             // hkv_ctx_create completed
    int pos_stride = 1;             // 0 with HKV_FLAG_SCALAR_POSITION
    float* prefill_ws = nullptr;    // [max_seq_new][kPrefillMaxSplits][H][HD+2] key-split partials of the prefill kernel
    int* prefill_counter = nullptr; // work counter of the two-tile prefill kernel (zeroed on the stream before each launch)
    int* prefill_row_parts = nullptr; // [max_seq_new][KVH]: partial rows per (query, kv head) under the equal-span schedule
    // host-buffer entry point staging
    __half *st_q = nullptr, *st_k = nullptr, *st_v = nullptr, *st_out = nullptr;
    // pipelined host op: a ring of staging sets, a stream for each copy direction
    struct HostSlot {
        __half *q = nullptr, *k = nullptr, *v = nullptr, *out = nullptr;
        cudaEvent_t in_done = nullptr, compute_done = nullptr, out_done = nullptr;
        bool used = false;
    };
    static constexpr int kHostSlots = 4;
    HostSlot host_slots[kHostSlots];
    cudaStream_t host_in = nullptr, host_out = nullptr;
    unsigned long long host_calls = 0;
    std::map<std::pair<const void*, const void*>, TmapPair> tmaps;   // keyed on the (k, v) plane pair
    std::string err;
    std::vector<double> plan_scratch;   // per-SM loads of the prefill split cost model
    // per-kernel timing (hkv_ctx_profile_begin/end)
    std::vector<cudaEvent_t> prof_events;  // 3 per timed call
    int prof_calls = 0, prof_max = 0;
};

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
                cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int fail(hkv_ctx* c, int code, const char* msg) {
    if (c) c->err = msg;
    return code;
}
int fail(hkv_ctx* c, int code, const std::string& msg) {
    if (c) c->err = msg;
    return code;
}
int fail_cuda(hkv_ctx* c, cudaError_t e, const char* where) {
    if (c) c->err = std::string(where) + ": " + cudaGetErrorString(e);
    return HKV_ERR_CUDA;
}

bool aligned(const void* p, size_t n) { return (reinterpret_cast<uintptr_t>(p) % n) == 0; }

int validate_geometry(const hkv_geometry* g, const char** why) {
    if (!g) { *why = "geometry is null"; return HKV_ERR_INVALID_ARG; }
    if (g->batch <= 0 || g->slots <= 0 || g->window_size < 0 || g->chunk_tiles < 0 ||
        g->batch_stride_elems < 0 || g->max_seq_new < 0) {
        *why = "batch/slots must be positive; window/chunk_tiles/stride non-negative";
        return HKV_ERR_INVALID_ARG;
    }
    // same guard as the reference op (kernels/register_kernels.cpp:858-861)
    if (g->head_dim <= 0 || g->head_dim > 512 || g->num_kv_heads <= 0 || g->num_heads <= 0 ||
        g->num_heads % g->num_kv_heads != 0) {
        *why = "unsupported head geometry";
        return HKV_ERR_GEOMETRY;
    }
    if (g->layout != HKV_LAYOUT_LINEAR && g->layout != HKV_LAYOUT_RING) {
        *why = "unknown layout";
        return HKV_ERR_INVALID_ARG;
    }
    if (g->kernel_select < 0 || g->kernel_select > 2) {
        *why = "unknown kernel_select";
        return HKV_ERR_INVALID_ARG;
    }
    if ((g->flags & ~(HKV_FLAG_SCALAR_POSITION | HKV_FLAG_APPEND_ONLY)) != 0 || g->tune_prefill_splits < 0 ||
        g->tune_prefill_kernel < 0 || g->tune_prefill_kernel > 2 || g->tune_tma_groups < 0 || g->tune_tma_groups > 3) {
        *why = "unknown flag or tuning override";
        return HKV_ERR_INVALID_ARG;
    }
    if (g->batch > 65535) { *why = "batch exceeds 65535"; return HKV_ERR_TOO_LARGE; }
    const long long dense = (long long)g->slots * g->num_kv_heads * g->head_dim;
    if (g->batch_stride_elems != 0 && g->batch_stride_elems < dense) {
        *why = "batch_stride_elems smaller than one sequence's plane";
        return HKV_ERR_INVALID_ARG;
    }
    if ((g->q_seq_stride_elems != 0 && g->q_seq_stride_elems < g->num_heads * g->head_dim) ||
        (g->new_kv_seq_stride_elems != 0 && g->new_kv_seq_stride_elems < g->num_kv_heads * g->head_dim) ||
        g->reserved[0] != 0) {
        *why = "q_seq_stride_elems / new_kv_seq_stride_elems smaller than one sequence's row, or a reserved field set";
        return HKV_ERR_INVALID_ARG;
    }
    if (g->shard_count > 1) {
        if (g->shard_rank < 0 || g->shard_rank >= g->shard_count || g->shard_block <= 0 ||
            g->shard_block % kTileRows != 0) {
            *why = "shard_rank/shard_block invalid (block must be a positive multiple of 64)";
            return HKV_ERR_INVALID_ARG;
        }
        if (g->layout == HKV_LAYOUT_RING) {
            *why = "ring layout cannot be sequence-sharded";
            return HKV_ERR_GEOMETRY;
        }
    }
    return HKV_OK;
}

bool tma_geometry_ok(const hkv_geometry& g) {
    const int G = g.num_heads / g.num_kv_heads;
    const bool hd_ok = g.head_dim == 64 || g.head_dim == 96 || g.head_dim == 128 || g.head_dim == 256;
    const long long bs = g.batch_stride_elems ? g.batch_stride_elems
                                              : (long long)g.slots * g.num_kv_heads * g.head_dim;
    return hd_ok && G <= 16 && g.batch <= kTmaMaxBatch && bs % 8 == 0;
}

int auto_chunk_tiles(const hkv_geometry& g, int sm_count) {
    int rows = g.slots;
    if (g.window_size > 0 && g.window_size < rows) rows = g.window_size + kTileRows;
    // Work items of `ct` tiles: about four items per SM keeps the persistent CTAs balanced while
    // the per-item cost (query fragments, warp merge, partial row) stays amortised; at most 128
    // partials per sequence bounds the serial merge loop of the combine kernel.
    const long long per_seq = (rows + kTileRows - 1) / kTileRows;
    const long long tiles = (long long)g.batch * g.num_kv_heads * per_seq;
    long long ct = tiles / ((long long)sm_count * 4);
    if (ct < (per_seq + 127) / 128) ct = (per_seq + 127) / 128;
    if (ct < 1) ct = 1;
    if (ct > 16) ct = 16;
    return (int)ct;
}

void fill_plan(const hkv_geometry& g, int sm_count, int& chunk_tiles, int& max_chunks) {
    chunk_tiles = g.chunk_tiles > 0 ? g.chunk_tiles : auto_chunk_tiles(g, sm_count > 0 ? sm_count : 148);
    const int tiles = (g.slots + kTileRows - 1) / kTileRows;
    max_chunks = (tiles + chunk_tiles - 1) / chunk_tiles;
    if (max_chunks < 1) max_chunks = 1;
}

size_t workspace_bytes_for(const hkv_geometry& g, int max_chunks) {
    return (size_t)g.batch * max_chunks * g.num_heads * (g.head_dim + 2) * sizeof(float);
}

// CTAs that share a span of the decode kernel's equal-span schedule. A gang of one CTA per kv head
// streams all heads of the same cache rows in step (a row holds every kv head side by side, so the
// gang reads whole rows together — measured: a gang of 4 for 32 kv heads, each CTA walking its span
// eight times, costs 9 %). CTAs beyond a whole number of gangs idle, so a gang may take two, four or
// eight heads per CTA when that leaves fewer than 6 % of the grid idle and one head per CTA does not.
int span_gang_for(int kv_heads, int grid) {
    int best = 1;
    double best_util = 0.0;
    for (int per_cta = 1; per_cta <= 8; per_cta *= 2) {
        if (kv_heads % per_cta != 0) break;
        const int gang = kv_heads / per_cta;
        if (gang > grid) continue;
        const double util = (double)(grid / gang) * gang / grid;
        if (util >= 0.94) return gang;
        if (util > best_util) { best_util = util; best = gang; }
    }
    return best;
}

// ---- TMA kernel table ------------------------------------------------------
typedef void (*TmaKernel)(const CUtensorMap, const CUtensorMap, const DecodeArgs, const int);

template <int HD>
TmaKernel pick_tma_hd(int nt, int groups, bool stale) {
    if (stale) {
        if (nt == 1) return groups == 1 ? hkv_decode_tma_kernel<HD, 1, 1, true> : hkv_decode_tma_kernel<HD, 1, 2, true>;
        return groups == 1 ? hkv_decode_tma_kernel<HD, 2, 1, true> : hkv_decode_tma_kernel<HD, 2, 2, true>;
    }
    if (nt == 1) return groups == 1 ? hkv_decode_tma_kernel<HD, 1, 1> : hkv_decode_tma_kernel<HD, 1, 2>;
    return groups == 1 ? hkv_decode_tma_kernel<HD, 2, 1> : hkv_decode_tma_kernel<HD, 2, 2>;
}
// A ring plane larger than its window, in whole tiles: the kernels that walk only the window's tiles.
bool tma_stale_ring(const hkv_geometry& g) {
    return g.layout == HKV_LAYOUT_RING && g.window_size > 0 && g.window_size < g.slots && g.slots % kTileRows == 0;
}
TmaKernel pick_tma(int HD, int nt, int groups, bool stale) {
    switch (HD) {
        case 64: return pick_tma_hd<64>(nt, groups, stale);
        case 96: return pick_tma_hd<96>(nt, groups, stale);
        case 128: return pick_tma_hd<128>(nt, groups, stale);
        case 256: return pick_tma_hd<256>(nt, groups, stale);
    }
    return nullptr;
}

// Encodes a tiled fp16 tensor map with 128-byte swizzle (rank 3 or 4).
int encode_f16_sw128(hkv_ctx* c, const void* base, int rank, const cuuint64_t* dims,
                     const cuuint64_t* strides, const cuuint32_t* box, CUtensorMap* out) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(c, HKV_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims,
                           strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[96];
        snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (CUresult %d)", (int)r);
        return fail(c, HKV_ERR_CUDA, buf);
    }
    return HKV_OK;
}

constexpr int kPrefillMaxSplits = 4;
// The decode kernel runs as two CTAs per SM unless that would give a sequence more spans than this.
constexpr int kMaxSpansPerSeqTwoCta = 40;

// Key tiles an item of `q_item` queries (item index qt) spans — the kernels' own arithmetic.
int prefill_span_tiles(const PrefillTcArgs& t, int q_item, int qt) {
    int kt0, ntot;
    prefill_item_tiles(t, q_item, prefill_tc_keys(t.HD), qt, kt0, ntot);
    return ntot;
}

// Key-range split count of the tensor-core prefill kernels. A kernel deals its work items
// (query tile or pair, kv head, split) round-robin to one CTA per SM, so the launch lasts as long
// as the most loaded CTA; this replays that deal with a per-item overhead (pipeline fill, Q load,
// output) and adds what the split costs (fp32 partials written and read back by the merge kernel).
// Costs are in microseconds, from timings of the kernels on B200.
int prefill_splits(const PrefillTcArgs& t, int HD, int q_item, double tile_us, int sm_count, bool have_ws,
                   int tune_splits, std::vector<double>& load, double* cost_out = nullptr) {
    if (cost_out) *cost_out = 1.0e30;
    const int max_s = have_ws ? kPrefillMaxSplits : 1;
    // No split may be empty: the split count is bounded by the SHORTEST span of any item. (With a
    // sliding window the spans differ by one tile from item to item, depending on how the window
    // falls on the tile grid; without one the first item has the shortest.)
    int min_span_tiles = 1 << 30;
    for (int qt = 0; qt < t.n_qtiles; ++qt) min_span_tiles = std::min(min_span_tiles, prefill_span_tiles(t, q_item, qt));
    if (tune_splits >= 1) return std::min(tune_splits, std::min(max_s, min_span_tiles));
    const double item_tiles = q_item > t.QT ? 5.0 : 6.0;
    const double row_bytes = (double)t.S_new * t.H * (HD + 2) * 4.0;
    int best = 1;
    double best_cost = 0.0;
    if (load.size() < (size_t)sm_count) load.resize((size_t)sm_count);   // grows once per context
    for (int s = 1; s <= max_s && s <= min_span_tiles; ++s) {
        const long long items = (long long)t.n_qtiles * t.KVH * s;
        const int grid = items < sm_count ? (int)items : sm_count;
        // The one-tile kernel deals items round-robin: replay the deal. The two-tile kernel hands
        // the next item (longest first) to whichever CTA is free: the full rounds even out, the
        // remainder lands on top — estimated in one pass, this runs on the host before every launch.
        const bool greedy = q_item > t.QT;
        if (!greedy) std::fill(load.begin(), load.begin() + sm_count, 0.0);
        const long long full = (items / grid) * grid;
        long long item = 0;
        double mx = 0.0, sum_full = 0.0, rem_first = 0.0;
        for (int qt = t.n_qtiles - 1; qt >= 0; --qt) {
            const int ntot = prefill_span_tiles(t, q_item, qt);
            const int base = ntot / s, rem = ntot % s;
            for (int kvh = 0; kvh < t.KVH; ++kvh)
                for (int sp = 0; sp < s; ++sp, ++item) {
                    const double w = (base + (sp < rem ? 1 : 0)) + item_tiles;
                    if (!greedy) load[(size_t)(item % grid)] += w;
                    else if (item < full) sum_full += w;
                    else if (w > rem_first) rem_first = w;
                }
        }
        if (greedy) mx = sum_full / grid + rem_first;
        else for (int i = 0; i < grid; ++i) mx = load[(size_t)i] > mx ? load[(size_t)i] : mx;
        double cost = mx * tile_us;
        if (s > 1) cost += 4.0 + 2.0 * s * row_bytes / 3.0e6;   // partials out and back at ~3 TB/s
        // (a split must promise 10 % with the self-balancing kernel: it runs its items a little less
        // efficiently than the model says, and the merge pass is pure overhead)
        if (s == 1 || cost < (greedy ? 0.90 : 0.97) * best_cost) { best = s; best_cost = cost; }
    }
    if (cost_out) *cost_out = best_cost;
    return best;
}

// Host-side plan of one tensor-core prefill launch: which kernel, how the chunk is cut into
// work items, how many key splits. Fills the shape fields of `t` (not the pointers). Pure
// arithmetic: no device is touched.
// Also decides the schedule of the two-tile kernel: equal spans (t.streamk, with `grid` CTAs) whenever
// partial rows can be kept and no split count is forced; otherwise whole items or uniform key splits.
void plan_prefill_tc(const hkv_geometry& g, int seq_new, int past_len, int sm_count, bool have_ws,
                     PrefillTcArgs& t, int& pair, int& min_span, int& grid, int& max_parts,
                     std::vector<double>& scratch) {
    const int G = g.num_heads / g.num_kv_heads, HD = g.head_dim;
    t.HD = HD;
    t.ring = g.layout == HKV_LAYOUT_RING ? 1 : 0;
    t.S_new = seq_new;
    t.past_len = past_len;
    t.H = g.num_heads;
    t.KVH = g.num_kv_heads;
    t.G = G;
    t.QT = kPfRows / G;
    // two query tiles per work item (hkv_prefill_tc2_kernel) unless the whole chunk fits one tile;
    // head_dim 256 always takes the one-tile kernel (its output alone fills half of tensor memory)
    pair = seq_new > t.QT ? 1 : 0;
    if (g.tune_prefill_kernel) pair = g.tune_prefill_kernel == 1 ? 0 : 1;
    if (HD == 256) pair = 0;
    const int q_item = pair ? 2 * t.QT : t.QT;
    t.n_qtiles = (seq_new + q_item - 1) / q_item;
    t.slots = g.slots;
    t.window = g.window_size;
    const int HDS = prefill_tc_staged_hd(HD);
    double tile_us = pair ? 0.85 + 0.85 * HDS / 128.0 : 0.60 + 0.95 * HDS / 128.0;   // per 128-row key tile of an item
    if (prefill_tc_keys(HD) == 64) tile_us *= 0.55;                                   // half-height tiles
    min_span = 1 << 30;
    int max_span = 0;
    long long total_tiles = 0;
    for (int qt = 0; qt < t.n_qtiles; ++qt) {
        const int n = prefill_span_tiles(t, q_item, qt);
        min_span = std::min(min_span, n);
        max_span = std::max(max_span, n);
        total_tiles += n;
    }
    total_tiles *= t.KVH;
    t.streamk = 0;
    t.sk_whole = 0;
    t.sk_grid = 0;
    t.part_stride = 1;
    t.row_parts = nullptr;
    double uniform_cost = 0.0;
    t.splits = prefill_splits(t, HD, q_item, tile_us, sm_count, have_ws, g.tune_prefill_splits, scratch, &uniform_cost);
    const long long n_items1 = (long long)t.n_qtiles * t.KVH;
    // (Measured: with fewer items than SMs uniform key splits do as well; with K/V planes beyond the L2
    // the spread start offsets of the spans cost the tile reuse that lockstep items get from it.)
    const double plane_mb = 4.0 * prefill_kv_valid(t) * t.KVH * HD / 1.0e6;
    if (pair && have_ws && g.tune_prefill_splits == 0 && t.n_qtiles <= kPf2MaxPairs && n_items1 > sm_count &&
        n_items1 % sm_count != 0 && plane_mb <= 100.0) {
        // Candidate: whole items for the full rounds of the grid, equal spans for the rest (items are
        // processed longest first, so the rest are the shortest). The spans shrink to fewer CTAs until
        // no item is cut into more parts than the workspace holds rows for.
        const long long whole = (n_items1 / sm_count) * sm_count;
        const double ov = 5.0;                       // tile steps a piece of work costs besides its key tiles
        double sum_whole = 0.0;
        long long tail_tiles = 0, idx = 0;
        int tail_max = 0;
        for (int qt = t.n_qtiles - 1; qt >= 0; --qt) {
            const int n = prefill_span_tiles(t, q_item, qt);
            for (int kvh = 0; kvh < t.KVH; ++kvh, ++idx) {
                if (idx < whole) sum_whole += n + ov;
                else { tail_tiles += n; tail_max = std::max(tail_max, n); }
            }
        }
        long long sg = std::min<long long>(sm_count, tail_tiles);
        int worst = kPrefillMaxSplits + 1;
        for (; sg >= 1; --sg) {
            if ((tail_max * sg + tail_tiles - 1) / tail_tiles > kPrefillMaxSplits) continue;   // cheap lower bound first
            worst = 1;
            long long P = 0;
            idx = 0;
            for (int qt = t.n_qtiles - 1; qt >= 0 && worst <= kPrefillMaxSplits; --qt) {
                const int n = prefill_span_tiles(t, q_item, qt);
                for (int kvh = 0; kvh < t.KVH; ++kvh, ++idx) {
                    if (idx < whole) continue;
                    worst = std::max(worst, prefill_span_owner(P + n - 1, tail_tiles, (int)sg) - prefill_span_owner(P, tail_tiles, (int)sg) + 1);
                    P += n;
                }
            }
            if (worst <= kPrefillMaxSplits) break;
        }
        if (sg >= 1 && worst <= kPrefillMaxSplits) {
            const double tail_rows_bytes = (double)(n_items1 - whole) / t.KVH * q_item * t.H * (HD + 2) * 4.0;
            const double sk_cost = (sum_whole / sm_count + (double)tail_tiles / sg + 2.0 * ov) * tile_us +
                                   4.0 + 2.0 * 2.0 * tail_rows_bytes / 3.0e6;   // partial rows out and back at ~3 TB/s
            if (sk_cost < 0.95 * uniform_cost) {
                t.streamk = 1;
                t.splits = 1;
                t.sk_whole = (int)whole;
                t.sk_grid = (int)sg;
                t.part_stride = kPrefillMaxSplits;
                grid = sm_count;
                max_parts = worst;
                return;
            }
        }
    }
    t.part_stride = t.splits;
    const long long items = (long long)t.n_qtiles * t.KVH * t.splits;
    grid = items < sm_count ? (int)items : sm_count;
    max_parts = t.splits;
}

// Geometries the tensor-core prefill kernels take: head_dim 64, 96, 128, 256; any group up to 128;
// linear planes, and ring planes whose row count is a whole number of key tiles.
bool prefill_tc_ok(const hkv_geometry& g) {
    const int G = g.num_heads / g.num_kv_heads;
    const bool hd_ok = g.head_dim == 64 || g.head_dim == 96 || g.head_dim == 128 || g.head_dim == 256;
    if (!hd_ok || G > 128 || g.shard_count > 1 || g.kernel_select == HKV_KERNEL_GENERIC) return false;
    if (g.layout == HKV_LAYOUT_RING && g.slots % prefill_tc_keys(g.head_dim) != 0) return false;
    const long long bs = g.batch_stride_elems ? g.batch_stride_elems : (long long)g.slots * g.num_kv_heads * g.head_dim;
    return bs % 8 == 0;
}

int encode_map(hkv_ctx* c, const void* base, CUtensorMap* out) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(c, HKV_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    const hkv_geometry& g = c->g;
    const int CW = tma_chunk_width(g.head_dim);
    cuuint64_t dims[4] = {(cuuint64_t)g.head_dim, (cuuint64_t)g.num_kv_heads, (cuuint64_t)g.slots,
                          (cuuint64_t)g.batch};
    cuuint64_t strides[3] = {(cuuint64_t)g.head_dim * 2, (cuuint64_t)g.num_kv_heads * g.head_dim * 2,
                             (cuuint64_t)c->batch_stride * 2};
    cuuint32_t box[4] = {(cuuint32_t)CW, 1u, (cuuint32_t)kTileRows, 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims,
                           strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CW == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[96];
        snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (CUresult %d)", (int)r);
        return fail(c, HKV_ERR_CUDA, buf);
    }
    return HKV_OK;
}

int get_maps(hkv_ctx* c, const void* k, const void* v, const TmapPair** out) {
    const std::pair<const void*, const void*> key(k, v);
    auto it = c->tmaps.find(key);
    if (it == c->tmaps.end()) {
        TmapPair p;
        int st = encode_map(c, k, &p.k);
        if (st) return st;
        st = encode_map(c, v, &p.v);
        if (st) return st;
        if (c->tmaps.size() > 4096) c->tmaps.clear();
        it = c->tmaps.emplace(key, p).first;
    }
    *out = &it->second;
    return HKV_OK;
}

// One launch of a tensor-core prefill kernel (+ its merge) for geometry `g`, which is the context's
// own or a view of it (the attend-before-append passes). `pass` == nullptr: the plain op.
struct PrefillPass {
    int key_limit;    // attend keys below this position only
    int out_part;     // partial slot (of out_parts) every row writes; the caller merges
    int out_parts;
};
int prefill_tc_launch(hkv_ctx* c, const hkv_geometry& g, const void* q, const void* k_plane, const void* v_plane, void* out,
                      int seq_new, int past_len, float scale, cudaStream_t st, const PrefillPass* pass) {
    const int HD = g.head_dim, G = g.num_heads / g.num_kv_heads, HDS = prefill_tc_staged_hd(HD), KEYS = prefill_tc_keys(HD);
    PrefillTcArgs t{};
    t.out = (__half*)out;
    t.status = c->d_status;
    t.key_limit = pass ? pass->key_limit : 0x7fffffff;
    t.out_part = pass ? pass->out_part : 0;
    t.out_parts = pass ? pass->out_parts : 0;
    int pair = 0, min_span = 0, grid = 0, max_parts = 0;
    plan_prefill_tc(g, seq_new, past_len, c->sm_count, !pass && c->prefill_ws != nullptr && seq_new <= c->g.max_seq_new, t, pair,
                    min_span, grid, max_parts, c->plan_scratch);
    if (t.splits > min_span || grid < 1 || max_parts > kPrefillMaxSplits)
        return fail(c, HKV_ERR_INVALID_ARG, "prefill: internal plan error (an empty key split or too many parts)");
    if (t.streamk) t.row_parts = c->prefill_row_parts;
    if (pass) t.part_stride = kPrefillMaxSplits;
    t.scale_log2 = scale * 1.4426950408889634f;
    t.part = c->prefill_ws;
    // Boxes are 64 halfs wide; a head_dim of 96 takes two, the second reaching past the tensor's
    // extent, where the copy engine fills zeros.
    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)g.num_heads, (cuuint64_t)seq_new};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)g.num_heads * HD * 2};
        cuuint32_t box[3] = {64u, (cuuint32_t)G, (cuuint32_t)t.QT};
        const int stt = encode_f16_sw128(c, q, 3, dims, strides, box, &mq);
        if (stt) return stt;
    }
    {
        cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)g.num_kv_heads, (cuuint64_t)g.slots, 1};
        cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)g.num_kv_heads * HD * 2,
                                 (cuuint64_t)g.slots * g.num_kv_heads * HD * 2};
        cuuint32_t box[4] = {64u, 1u, (cuuint32_t)KEYS, 1u};
        int stt = encode_f16_sw128(c, k_plane, 4, dims, strides, box, &mk);
        if (stt) return stt;
        stt = encode_f16_sw128(c, v_plane, 4, dims, strides, box, &mv);
        if (stt) return stt;
    }
    t.item_counter = c->prefill_counter;
    if (pair) {
        const cudaError_t me = cudaMemsetAsync(c->prefill_counter, 0, sizeof(int), st);
        if (me != cudaSuccess) return fail_cuda(c, me, "cudaMemsetAsync(prefill work counter)");
        const size_t smem = prefill_tc2_smem_bytes(HDS);
        if (HDS == 64) hkv_prefill_tc2_kernel<64><<<grid, kPf2Threads, smem, st>>>(mq, mk, mv, t);
        else hkv_prefill_tc2_kernel<128><<<grid, kPf2Threads, smem, st>>>(mq, mk, mv, t);
    } else {
        const size_t smem = prefill_tc_smem_bytes(HDS);
        if (HDS == 64) hkv_prefill_tc_kernel<64, 128><<<grid, kPfThreads, smem, st>>>(mq, mk, mv, t);
        else if (HDS == 128) hkv_prefill_tc_kernel<128, 128><<<grid, kPfThreads, smem, st>>>(mq, mk, mv, t);
        else hkv_prefill_tc_kernel<256, 64><<<grid, kPfThreads, smem, st>>>(mq, mk, mv, t);
    }
    if (!pass && (t.splits > 1 || (t.streamk && max_parts > 1))) {
        // merge the key-range partials of every (query, head) that has more than one
        const long long rows = (long long)seq_new * g.num_heads;
        const unsigned cgrid = (unsigned)((rows + 7) / 8);
        hkv_prefill_combine_kernel<<<cgrid, 256, 0, st>>>(c->prefill_ws, (__half*)out, rows, g.num_heads, HD, t.splits,
                                                         t.part_stride, t.row_parts, G);
    }
    const cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? HKV_OK : fail_cuda(c, e, "prefill launch");
}

SeqMap make_map(const hkv_geometry& g) {
    SeqMap m;
    m.slots = g.slots;
    m.layout = g.layout;
    m.window = g.window_size;
    m.shard_rank = g.shard_count > 1 ? g.shard_rank : 0;
    m.shard_count = g.shard_count > 1 ? g.shard_count : 1;
    m.shard_block = g.shard_count > 1 ? g.shard_block : kTileRows;
    return m;
}

int launch_append(hkv_ctx* c, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                  const int32_t* d_pos, int pos_bias, int host_pos, int seq_new, cudaStream_t st, bool dense = false) {
    if (!k_new || !v_new || !k_cache || !v_cache) return fail(c, HKV_ERR_INVALID_ARG, "append: null tensor");
    if (seq_new < 0) return fail(c, HKV_ERR_INVALID_ARG, "append: negative seq_new");
    const long long natural = (long long)c->g.num_kv_heads * c->g.head_dim;
    if (!dense && seq_new > 1 && c->new_stride != natural)
        return fail(c, HKV_ERR_GEOMETRY, "append: new_kv_seq_stride_elems describes one new token per sequence; seq_new > 1 takes dense tensors");
    if (!aligned(k_new, 2) || !aligned(v_new, 2) || !aligned(k_cache, 2) || !aligned(v_cache, 2))
        return fail(c, HKV_ERR_ALIGNMENT, "append: fp16 pointer not 2-byte aligned");
    if (seq_new == 0) return HKV_OK;
    AppendArgs a{};
    a.k_new = (const __half*)k_new;
    a.v_new = (const __half*)v_new;
    a.k_cache = (__half*)k_cache;
    a.v_cache = (__half*)v_cache;
    a.d_pos = d_pos;
    a.pos_stride = c->pos_stride;
    a.host_pos = host_pos;
    a.pos_bias = pos_bias;
    a.map = c->map;
    a.B = c->g.batch;
    a.S = seq_new;
    a.row_elems = c->g.num_kv_heads * c->g.head_dim;
    a.batch_stride = c->batch_stride;
    a.src_stride = (dense || seq_new > 1) ? (long long)seq_new * a.row_elems : c->new_stride;
    const bool vec = aligned(k_new, 16) && aligned(v_new, 16) && aligned(k_cache, 16) &&
                     aligned(v_cache, 16) && a.row_elems % 8 == 0 && c->batch_stride % 8 == 0 && a.src_stride % 8 == 0;
    const long long pieces = 2ll * a.B * a.S * (vec ? a.row_elems / 8 : a.row_elems);
    long long blocks = (pieces + 255) / 256;
    const long long cap = (long long)c->sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (vec) hkv_append_kernel<uint4><<<(unsigned)blocks, 256, 0, st>>>(a);
    else hkv_append_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(a);
    return HKV_OK;
}

// Decode into the workspace; `fused` appends k_new/v_new at position total-1.
int launch_decode(hkv_ctx* c, const void* q, const void* k_new, const void* v_new, void* k_cache,
                  void* v_cache, const int32_t* d_total, int pos_is_index, int host_len, float scale,
                  cudaStream_t st, bool* used_tma, bool dense = false) {
    *used_tma = false;
    const hkv_geometry& g = c->g;
    if (!q || !k_cache || !v_cache) return fail(c, HKV_ERR_INVALID_ARG, "decode: null tensor");
    if (!aligned(q, 2) || !aligned(k_cache, 2) || !aligned(v_cache, 2))
        return fail(c, HKV_ERR_ALIGNMENT, "decode: fp16 pointer not 2-byte aligned");
    if (!std::isfinite(scale)) return fail(c, HKV_ERR_INVALID_ARG, "decode: scale is not finite");
    const bool fused = k_new != nullptr;
    if (fused && !v_new) return fail(c, HKV_ERR_INVALID_ARG, "decode: k_new without v_new");

    DecodeArgs a{};
    a.q = (const __half*)q;
    a.k_cache = (const __half*)k_cache;
    a.v_cache = (const __half*)v_cache;
    a.k_new = nullptr;
    a.v_new = nullptr;
    a.k_cache_w = (__half*)k_cache;
    a.v_cache_w = (__half*)v_cache;
    a.part = c->workspace;
    a.span_part = nullptr;
    a.gpre = nullptr;
    a.span_gang = 1;
    a.total = d_total;
    a.status = c->d_status;
    a.map = c->map;
    a.B = g.batch;
    a.H = g.num_heads;
    a.KVH = g.num_kv_heads;
    a.HD = g.head_dim;
    a.chunk_tiles = c->chunk_tiles;
    a.max_chunks = c->max_chunks;
    a.pos_is_index = pos_is_index;
    a.pos_stride = c->pos_stride;
    a.host_len = host_len;
    a.batch_stride = c->batch_stride;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.q_stride = dense ? (long long)g.num_heads * g.head_dim : c->q_stride;
    a.new_stride = dense ? (long long)g.num_kv_heads * g.head_dim : c->new_stride;

    bool use_tma = c->kernel == HKV_KERNEL_TMA && aligned(q, 16) && aligned(k_cache, 16) &&
                   aligned(v_cache, 16) && a.q_stride % 8 == 0 &&
                   (!fused || (aligned(k_new, 16) && aligned(v_new, 16) && a.new_stride % 8 == 0));
    if (!use_tma && g.kernel_select == HKV_KERNEL_TMA)
        return fail(c, HKV_ERR_ALIGNMENT, "decode: TMA kernel requires 16-byte aligned tensors");

    if (use_tma) {
        const TmapPair* maps = nullptr;
        const int stt = get_maps(c, k_cache, v_cache, &maps);
        if (stt) return stt;
        if (fused) { a.k_new = (const __half*)k_new; a.v_new = (const __half*)v_new; }
        const int nt = (c->G + 7) / 8;
        const int groups = c->tma_groups == 2 ? 2 : 1;
        TmaKernel kern = pick_tma(g.head_dim, nt, groups, tma_stale_ring(g));
        a.span_part = c->span_ws;
        a.gpre = c->span_gpre;
        a.span_gang = c->span_gang;
        const int threads = (groups * 4 + 1) * 32;
        kern<<<c->tma_grid, threads, c->plan.bytes, st>>>(maps->k, maps->v, a, c->plan.stages);
        *used_tma = true;
    } else {
        if (fused) {
            // generic path: append first (its own launch), then attend; the new row sits at
            // position total - 1 when the array holds attended lengths
            if (!d_total) return fail(c, HKV_ERR_INVALID_ARG, "fused decode needs device positions");
            const int stt = launch_append(c, k_new, v_new, k_cache, v_cache, d_total, pos_is_index ? 0 : -1, 0, 1, st, dense);
            if (stt) return stt;
        }
        dim3 grid((unsigned)c->max_chunks, (unsigned)g.num_heads, (unsigned)g.batch);
        hkv_decode_generic_kernel<<<grid, kGenWarps * 32, 0, st>>>(a);
    }
    return HKV_OK;
}

constexpr size_t kMailboxHeaderBytes = 512;   // 64 flag words + 64 state words

int check_exchange(hkv_ctx* c, const hkv_exchange* x, const char* who) {
    if (!x) return fail(c, HKV_ERR_INVALID_ARG, std::string(who) + ": null exchange");
    if (x->world < 1 || x->world > HKV_MAX_PEERS || x->rank < 0 || x->rank >= x->world)
        return fail(c, HKV_ERR_INVALID_ARG, std::string(who) + ": rank/world out of range (at most " +
                                                std::to_string(HKV_MAX_PEERS) + " ranks)");
    const int shards = c->g.shard_count > 1 ? c->g.shard_count : 1;
    if (x->world != shards || (shards > 1 && x->rank != c->g.shard_rank))
        return fail(c, HKV_ERR_GEOMETRY, std::string(who) + ": exchange rank/world differ from the context's shard_rank/shard_count");
    for (int r = 0; r < x->world; ++r) {
        if (!x->mailbox[r]) return fail(c, HKV_ERR_INVALID_ARG, std::string(who) + ": null mailbox");
        if (!aligned(x->mailbox[r], 256)) return fail(c, HKV_ERR_ALIGNMENT, std::string(who) + ": mailbox not 256-byte aligned");
    }
    if (x->wait_limit_ms < 0 || x->wait_limit_ms > 10000)
        return fail(c, HKV_ERR_INVALID_ARG, std::string(who) + ": wait_limit_ms outside 0..10000");
    return HKV_OK;
}

int launch_combine(hkv_ctx* c, const float* part, long long stride_b, long long stride_c,
                   const int32_t* d_total, int pos_is_index, int host_len, int fixed_count, void* out,
                   float* out_partial, cudaStream_t st, bool span = false, const hkv_exchange* x = nullptr) {
    CombineArgs a{};
    if (x) {
        // mailbox: 64 flag words, 64 state words, then [2][batch*heads*(head_dim+2)] floats
        uint8_t* mine = (uint8_t*)x->mailbox[x->rank];
        a.pub_n = x->world;
        a.pub_part = (float*)(mine + kMailboxHeaderBytes);
        a.pub_parity_stride = (long long)c->g.batch * c->g.num_heads * (c->g.head_dim + 2);
        a.pub_state = (const uint32_t*)(mine + kMailboxHeaderBytes / 2);
    }
    a.gpre = span ? c->span_gpre : nullptr;
    a.span_spans = span ? c->tma_grid / c->span_gang : 0;
    a.B = c->g.batch;
    a.part = part;
    a.stride_b = stride_b;
    a.stride_c = stride_c;
    a.total = d_total;
    a.pos_is_index = pos_is_index;
    a.pos_stride = c->pos_stride;
    a.host_len = host_len;
    a.fixed_count = fixed_count;
    a.map = c->map;
    a.chunk_tiles = c->chunk_tiles;
    a.H = c->g.num_heads;
    a.HD = c->g.head_dim;
    a.out = (__half*)out;
    a.out_partial = out_partial;
    dim3 grid((unsigned)c->g.num_heads, (unsigned)c->g.batch);
    // Two merge kernels, chosen by host constants of the context (so a captured graph never changes
    // kernel): with few (sequence, head) rows and many partials per row the merge is latency-bound
    // and the warp-dealt kernel wins (batch 1-8: +5 %); with many rows the one-thread-per-dimension
    // kernel does (batch 32-64: +2 % of the step).
    // partials a row can have: the chunks of a full plane, or (equal spans) about spans / batch + 1
    const int most = fixed_count > 0 ? fixed_count
                     : span ? (c->tma_grid / c->span_gang) / c->g.batch + 1 : c->max_chunks;
    const long long rows = (long long)grid.x * grid.y;
    if (rows <= 2LL * c->sm_count && most > 8) hkv_combine_kernel<<<grid, kCombineThreads, 0, st>>>(a);
    else hkv_combine_few_kernel<<<grid, 128, 0, st>>>(a);
    return HKV_OK;
}

int decode_full(hkv_ctx* c, const void* q, const void* k_new, const void* v_new, void* k_cache,
                void* v_cache, void* out, float* out_partial, const int32_t* d_total,
                int pos_is_index, int host_len, float scale, cudaStream_t st, const hkv_exchange* x = nullptr,
                bool dense = false) {
    if (!c->workspace) return fail(c, HKV_ERR_WORKSPACE, "decode: the context was created append-only");
    if (!out && !out_partial && !x) return fail(c, HKV_ERR_INVALID_ARG, "decode: null output");
    if (out && !aligned(out, 2)) return fail(c, HKV_ERR_ALIGNMENT, "decode: out not 2-byte aligned");
    const bool timed = c->prof_calls < c->prof_max;
    cudaEvent_t* ev = timed ? &c->prof_events[(size_t)c->prof_calls * 3] : nullptr;
    if (timed) cudaEventRecord(ev[0], st);
    bool used_tma = false;
    int stt = launch_decode(c, q, k_new, v_new, k_cache, v_cache, d_total, pos_is_index, host_len, scale, st, &used_tma, dense);
    if (stt) return stt;
    if (timed) cudaEventRecord(ev[1], st);
    const long long PW = c->g.head_dim + 2;
    stt = launch_combine(c, used_tma ? c->span_ws : c->workspace, (long long)c->max_chunks * c->g.num_heads * PW,
                         (long long)c->g.num_heads * PW, d_total, pos_is_index, host_len, 0, out, out_partial,
                         st, used_tma, x);
    if (stt) return stt;
    if (timed) {
        cudaEventRecord(ev[2], st);
        ++c->prof_calls;
    }
    const cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return fail_cuda(c, e, "decode launch");
    return HKV_OK;
}

}  // namespace

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
extern "C" {

int hkv_abi_version(void) { return HKV_ABI_VERSION; }

const char* hkv_status_string(int s) {
    switch (s) {
        case HKV_OK: return "ok";
        case HKV_ERR_INVALID_ARG: return "invalid argument";
        case HKV_ERR_GEOMETRY: return "unsupported geometry";
        case HKV_ERR_ALIGNMENT: return "misaligned pointer or stride";
        case HKV_ERR_CUDA: return "CUDA call failed";
        case HKV_ERR_NO_DEVICE: return "no usable B200-class CUDA device";
        case HKV_ERR_WORKSPACE: return "workspace too small";
        case HKV_ERR_TOO_LARGE: return "size exceeds a documented maximum";
        case HKV_ERR_DEVICE_FAULT: return "device status word reports a fault";
    }
    return "unknown status";
}

size_t hkv_workspace_bytes(const hkv_geometry* g) {
    const char* why;
    if (validate_geometry(g, &why) != HKV_OK) return 0;
    int sm = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sm = v;
    } else {
        cudaGetLastError();
    }
    int ct, mc;
    fill_plan(*g, sm, ct, mc);
    return workspace_bytes_for(*g, mc);
}

size_t hkv_partial_floats(const hkv_geometry* g) { return g ? (size_t)g->head_dim + 2 : 0; }

int hkv_ctx_create(hkv_ctx** out, const hkv_geometry* geometry) {
    if (!out) return HKV_ERR_INVALID_ARG;
    *out = nullptr;
    const char* why = "";
    const int vst = validate_geometry(geometry, &why);
    hkv_ctx* c = new (std::nothrow) hkv_ctx();
    if (!c) return HKV_ERR_CUDA;
    *out = c;  // returned even on failure so the caller can read the message; destroy it
    if (vst) return fail(c, vst, why);
    c->g = *geometry;

    int dev = 0, ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        return fail(c, HKV_ERR_NO_DEVICE, "no CUDA device");
    }
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda(c, e, "cudaGetDevice");
    int major = 0, sm = 0, optin = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (major != 10) return fail(c, HKV_ERR_NO_DEVICE, "device is not compute capability 10.x (built for sm_100a only)");
    c->device = dev;
    c->sm_count = sm;
    c->smem_optin = (size_t)optin;
    c->G = geometry->num_heads / geometry->num_kv_heads;
    c->batch_stride = geometry->batch_stride_elems
                          ? geometry->batch_stride_elems
                          : (long long)geometry->slots * geometry->num_kv_heads * geometry->head_dim;
    c->map = make_map(*geometry);
    c->pos_stride = (geometry->flags & HKV_FLAG_SCALAR_POSITION) ? 0 : 1;
    c->q_stride = geometry->q_seq_stride_elems ? geometry->q_seq_stride_elems : (long long)geometry->num_heads * geometry->head_dim;
    c->new_stride = geometry->new_kv_seq_stride_elems ? geometry->new_kv_seq_stride_elems
                                                      : (long long)geometry->num_kv_heads * geometry->head_dim;
    fill_plan(*geometry, sm, c->chunk_tiles, c->max_chunks);
    e = cudaMalloc(&c->d_status, sizeof(int32_t));
    if (e != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(status)");
    e = cudaMemset(c->d_status, 0, sizeof(int32_t));
    if (e != cudaSuccess) return fail_cuda(c, e, "cudaMemset(status)");
    if (geometry->flags & HKV_FLAG_APPEND_ONLY) {   // no attention: no workspaces, no kernel opt-ins
        c->ready = true;
        return HKV_OK;
    }

    // kernel choice
    const bool tma_ok = tma_geometry_ok(*geometry);
    if (geometry->kernel_select == HKV_KERNEL_TMA && !tma_ok)
        return fail(c, HKV_ERR_GEOMETRY, "TMA kernel needs head_dim in {64,96,128,256}, group <= 16, stride % 8 == 0");
    c->kernel = (geometry->kernel_select != HKV_KERNEL_GENERIC && tma_ok) ? HKV_KERNEL_TMA
                                                                           : HKV_KERNEL_GENERIC;
    if (c->kernel == HKV_KERNEL_TMA) {
        // Two shapes of the same kernel (hkv_decode_tma.cuh): one CTA per SM with two consumer groups,
        // or two CTAs per SM with one group and half the ring each.
        int sm_total = 0;
        cudaDeviceGetAttribute(&sm_total, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
        const size_t half_budget = sm_total > 4096 ? (size_t)sm_total / 2 - 2048 : 0;   // two CTAs + the runtime's reserve
        // Two CTAs per SM stream a little faster (7.1 against 6.6 TB/s at batch 64) and hide each other's
        // merges; they also double the spans, and with them the partials the merge kernel walks per
        // sequence — which is what a launch of one or two sequences spends its time on.
        const int spans_two = 2 * sm / span_gang_for(geometry->num_kv_heads, 2 * sm);
        c->tma_groups = geometry->tune_tma_groups ? geometry->tune_tma_groups : (spans_two / geometry->batch > kMaxSpansPerSeqTwoCta ? 2 : 1);
        if (c->tma_groups == 1) {
            c->plan = tma_plan(geometry->head_dim, c->G, 4, geometry->batch, half_budget);
            if (c->plan.stages < 2) c->tma_groups = 2;   // tiles too large for half an SM's shared memory
        }
        if (c->tma_groups == 2) c->plan = tma_plan(geometry->head_dim, c->G, 8, geometry->batch, c->smem_optin);
        if ((c->plan.stages < 2 && c->tma_groups == 2) || c->tma_groups == 3) {
            c->tma_groups = 0;    // one CTA per SM, one consumer group, the whole shared memory
            c->plan = tma_plan(geometry->head_dim, c->G, 4, geometry->batch, c->smem_optin);
        }
        if (c->plan.stages < 2) {
            if (geometry->kernel_select == HKV_KERNEL_TMA)
                return fail(c, HKV_ERR_GEOMETRY, "TMA kernel: shared memory too small for two stages");
            c->kernel = HKV_KERNEL_GENERIC;
        } else {
            if (!encode_tiled_fn()) return fail(c, HKV_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
            TmaKernel kern = pick_tma(geometry->head_dim, (c->G + 7) / 8, c->tma_groups == 2 ? 2 : 1, tma_stale_ring(*geometry));
            // the attribute belongs to the kernel, not to this context: keep it at the device
            // maximum so that contexts with different plans never lower it for each other
            e = cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)c->smem_optin);
            if (e != cudaSuccess) return fail_cuda(c, e, "cudaFuncSetAttribute(shared memory)");
        }
    }

    if (prefill_tc_ok(*geometry)) {
        const int hds = prefill_tc_staged_hd(geometry->head_dim);
        const void* pk = hds == 64 ? (const void*)hkv_prefill_tc_kernel<64, 128>
                       : hds == 128 ? (const void*)hkv_prefill_tc_kernel<128, 128>
                                    : (const void*)hkv_prefill_tc_kernel<256, 64>;
        e = cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_tc_smem_bytes(hds));
        if (e != cudaSuccess) return fail_cuda(c, e, "cudaFuncSetAttribute(prefill shared memory)");
        if (hds != 256) {
            const void* pk2 = hds == 64 ? (const void*)hkv_prefill_tc2_kernel<64> : (const void*)hkv_prefill_tc2_kernel<128>;
            e = cudaFuncSetAttribute(pk2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_tc2_smem_bytes(hds));
            if (e != cudaSuccess) return fail_cuda(c, e, "cudaFuncSetAttribute(prefill shared memory)");
        }
    }
    if (prefill_tc_ok(*geometry)) {
        e = cudaMalloc(&c->prefill_counter, sizeof(int));
        if (e != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(prefill work counter)");
    }
    if (prefill_tc_ok(*geometry) && geometry->max_seq_new > 0) {
        const size_t nb = (size_t)geometry->max_seq_new * kPrefillMaxSplits * geometry->num_heads *
                          (geometry->head_dim + 2) * sizeof(float);
        e = cudaMalloc(&c->prefill_ws, nb);
        if (e != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(prefill workspace)");
        e = cudaMalloc(&c->prefill_row_parts, sizeof(int) * (size_t)geometry->max_seq_new * geometry->num_kv_heads);
        if (e != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(prefill row counts)");
    }
    c->workspace_bytes = workspace_bytes_for(*geometry, c->max_chunks);
    e = cudaMalloc(&c->workspace, c->workspace_bytes);
    if (e != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(workspace)");
    if (c->kernel == HKV_KERNEL_TMA) {
        // Equal-span schedule: one or two persistent CTAs per SM, in gangs that share a span with one
        // share of the kv heads each; one partial row set per (span, sequence) piece.
        c->tma_grid = (c->tma_groups == 1 ? 2 : 1) * sm;
        c->span_gang = span_gang_for(geometry->num_kv_heads, c->tma_grid);
        const size_t slots = (size_t)c->tma_grid / c->span_gang + geometry->batch;
        e = cudaMalloc(&c->span_ws, slots * geometry->num_heads * (geometry->head_dim + 2) * sizeof(float));
        if (e != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(span workspace)");
        e = cudaMalloc(&c->span_gpre, sizeof(int) * ((size_t)geometry->batch + 1));
        if (e != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(tile table)");
    }
    c->ready = true;
    return HKV_OK;
}

int hkv_ctx_destroy(hkv_ctx* c) {
    if (!c) return HKV_OK;
    if (c->workspace) cudaFree(c->workspace);
    if (c->span_ws) cudaFree(c->span_ws);
    if (c->span_gpre) cudaFree(c->span_gpre);
    if (c->d_status) cudaFree(c->d_status);
    if (c->prefill_ws) cudaFree(c->prefill_ws);
    if (c->prefill_counter) cudaFree(c->prefill_counter);
    if (c->prefill_row_parts) cudaFree(c->prefill_row_parts);
    if (c->st_q) cudaFree(c->st_q);
    if (c->st_k) cudaFree(c->st_k);
    if (c->st_v) cudaFree(c->st_v);
    if (c->st_out) cudaFree(c->st_out);
    if (c->host_in) cudaStreamSynchronize(c->host_in);
    if (c->host_out) cudaStreamSynchronize(c->host_out);
    for (hkv_ctx::HostSlot& h : c->host_slots) {
        if (h.q) cudaFree(h.q);
        if (h.k) cudaFree(h.k);
        if (h.v) cudaFree(h.v);
        if (h.out) cudaFree(h.out);
        if (h.in_done) cudaEventDestroy(h.in_done);
        if (h.compute_done) cudaEventDestroy(h.compute_done);
        if (h.out_done) cudaEventDestroy(h.out_done);
    }
    if (c->host_in) cudaStreamDestroy(c->host_in);
    if (c->host_out) cudaStreamDestroy(c->host_out);
    for (cudaEvent_t e : c->prof_events) cudaEventDestroy(e);
    delete c;
    return HKV_OK;
}

const char* hkv_ctx_last_error(const hkv_ctx* c) { return c ? c->err.c_str() : "null context"; }
int hkv_ctx_kernel(const hkv_ctx* c) { return c ? c->kernel : 0; }
int hkv_ctx_launches_per_decode(const hkv_ctx* c) { return c ? 2 : 0; }

// Every launch entry point: the context must be complete and the CURRENT device must be the one
// it was created on (its workspace, status word, tensor maps and shared-memory opt-ins live there).
static int check_ctx(hkv_ctx* c) {
    if (!c) return HKV_ERR_INVALID_ARG;
    if (!c->ready) return fail(c, HKV_ERR_INVALID_ARG, "context not initialised");
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return fail(c, HKV_ERR_CUDA, "cudaGetDevice failed");
    }
    if (dev != c->device) {
        char buf[96];
        snprintf(buf, sizeof buf, "context belongs to device %d, current device is %d", c->device, dev);
        return fail(c, HKV_ERR_INVALID_ARG, buf);
    }
    return HKV_OK;
}
#define HKV_CHECK_CTX(c)                        \
    do {                                        \
        const int chk_ = check_ctx(c);          \
        if (chk_ != HKV_OK) return chk_;        \
    } while (0)

int hkv_ctx_device_status(hkv_ctx* c, void* stream, int32_t* status_out) {
    if (!c || !status_out) return HKV_ERR_INVALID_ARG;
    HKV_CHECK_CTX(c);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail_cuda(c, e, "cudaStreamSynchronize");
    e = cudaMemcpy(status_out, c->d_status, sizeof(int32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(c, e, "cudaMemcpy(status)");
    if (*status_out != 0) {
        cudaMemset(c->d_status, 0, sizeof(int32_t));
        return fail(c, HKV_ERR_DEVICE_FAULT, "device status word is non-zero");
    }
    return HKV_OK;
}


int hkv_append(hkv_ctx* c, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
               const int32_t* d_cache_pos, int32_t seq_new, void* stream) {
    HKV_CHECK_CTX(c);
    if (!d_cache_pos) return fail(c, HKV_ERR_INVALID_ARG, "append: null position array");
    const int st = launch_append(c, k_new, v_new, k_cache, v_cache, d_cache_pos, 0, 0, seq_new,
                                 (cudaStream_t)stream);
    if (st) return st;
    const cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? HKV_OK : fail_cuda(c, e, "append launch");
}

int hkv_append_at(hkv_ctx* c, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                  int32_t position, int32_t seq_new, void* stream) {
    HKV_CHECK_CTX(c);
    if (position < 0) return fail(c, HKV_ERR_INVALID_ARG, "append: negative position");
    const int st = launch_append(c, k_new, v_new, k_cache, v_cache, nullptr, 0, position, seq_new,
                                 (cudaStream_t)stream);
    if (st) return st;
    const cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? HKV_OK : fail_cuda(c, e, "append launch");
}

int hkv_decode_attention(hkv_ctx* c, const void* q, const void* k_cache, const void* v_cache,
                         void* out, const int32_t* d_total_seq, float scale, void* stream) {
    HKV_CHECK_CTX(c);
    if (!d_total_seq) return fail(c, HKV_ERR_INVALID_ARG, "decode: null length array");
    return decode_full(c, q, nullptr, nullptr, const_cast<void*>(k_cache), const_cast<void*>(v_cache),
                       out, nullptr, d_total_seq, 0, 0, scale, (cudaStream_t)stream);
}

int hkv_decode_attention_len(hkv_ctx* c, const void* q, const void* k_cache, const void* v_cache,
                             void* out, int32_t seq_len, float scale, void* stream) {
    HKV_CHECK_CTX(c);
    if (seq_len < 0) return fail(c, HKV_ERR_INVALID_ARG, "decode: negative seq_len");
    // the length is a kernel argument: nothing shared between calls, nothing to copy
    return decode_full(c, q, nullptr, nullptr, const_cast<void*>(k_cache), const_cast<void*>(v_cache),
                       out, nullptr, nullptr, 0, seq_len, scale, (cudaStream_t)stream);
}

int hkv_append_decode_attention(hkv_ctx* c, const void* q, const void* k_new, const void* v_new,
                                void* k_cache, void* v_cache, void* out,
                                const int32_t* d_cache_pos, float scale, void* stream) {
    HKV_CHECK_CTX(c);
    if (!k_new || !v_new) return fail(c, HKV_ERR_INVALID_ARG, "fused decode: null k_new/v_new");
    if (!aligned(k_new, 2) || !aligned(v_new, 2))
        return fail(c, HKV_ERR_ALIGNMENT, "fused decode: fp16 pointer not 2-byte aligned");
    if (!d_cache_pos) return fail(c, HKV_ERR_INVALID_ARG, "fused decode: null position array");
    return decode_full(c, q, k_new, v_new, k_cache, v_cache, out, nullptr, d_cache_pos, 1, 0, scale,
                       (cudaStream_t)stream);
}

int hkv_decode_partials(hkv_ctx* c, const void* q, const void* k_new, const void* v_new,
                        void* k_cache, void* v_cache, float* partial_out,
                        const int32_t* d_total_seq, float scale, void* stream) {
    HKV_CHECK_CTX(c);
    if (!partial_out) return fail(c, HKV_ERR_INVALID_ARG, "decode_partials: null output");
    if (!d_total_seq) return fail(c, HKV_ERR_INVALID_ARG, "decode_partials: null length array");
    if (k_new && !v_new) return fail(c, HKV_ERR_INVALID_ARG, "decode_partials: k_new without v_new");
    if (k_new && (!aligned(k_new, 2) || !aligned(v_new, 2)))
        return fail(c, HKV_ERR_ALIGNMENT, "decode_partials: fp16 pointer not 2-byte aligned");
    // d_total_seq holds attended lengths, so the new row sits at position total - 1. Only the rank
    // that owns that position stages and stores it (slot_of_pos is -1 elsewhere): the decode kernel
    // patches its tile, exactly as in hkv_append_decode_attention — no separate append launch.
    return decode_full(c, q, k_new, v_new, k_cache, v_cache, nullptr, partial_out, d_total_seq, 0, 0,
                       scale, (cudaStream_t)stream);
}

int hkv_combine_partials(hkv_ctx* c, const float* partials, int32_t num_parts, void* out,
                         void* stream) {
    HKV_CHECK_CTX(c);
    if (!partials || !out || num_parts <= 0) return fail(c, HKV_ERR_INVALID_ARG, "combine: bad arguments");
    if (!aligned(out, 2)) return fail(c, HKV_ERR_ALIGNMENT, "combine: out not 2-byte aligned");
    const long long PW = c->g.head_dim + 2;
    const int st = launch_combine(c, partials, (long long)c->g.num_heads * PW,
                                  (long long)c->g.batch * c->g.num_heads * PW, nullptr, 0, 0, num_parts,
                                  out, nullptr, (cudaStream_t)stream);
    if (st) return st;
    const cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? HKV_OK : fail_cuda(c, e, "combine launch");
}

int hkv_exchange_bytes(const hkv_ctx* c, int32_t world, size_t* bytes_out) {
    if (!c || !bytes_out || world < 1 || world > HKV_MAX_PEERS) return HKV_ERR_INVALID_ARG;
    *bytes_out = kMailboxHeaderBytes + 2ull * c->g.batch * c->g.num_heads * (size_t)(c->g.head_dim + 2) * sizeof(float);
    return HKV_OK;
}

int hkv_decode_partials_publish(hkv_ctx* c, const void* q, const void* k_new, const void* v_new,
                             void* k_cache, void* v_cache, const hkv_exchange* exchange,
                             const int32_t* d_total_seq, float scale, void* stream) {
    HKV_CHECK_CTX(c);
    const int stx = check_exchange(c, exchange, "decode_partials_publish");
    if (stx) return stx;
    if (!d_total_seq) return fail(c, HKV_ERR_INVALID_ARG, "decode_partials_publish: null length array");
    if (k_new && !v_new) return fail(c, HKV_ERR_INVALID_ARG, "decode_partials_publish: k_new without v_new");
    if (k_new && (!aligned(k_new, 2) || !aligned(v_new, 2)))
        return fail(c, HKV_ERR_ALIGNMENT, "decode_partials_publish: fp16 pointer not 2-byte aligned");
    return decode_full(c, q, k_new, v_new, k_cache, v_cache, nullptr, nullptr, d_total_seq, 0, 0, scale,
                       (cudaStream_t)stream, exchange);
}

int hkv_merge_published(hkv_ctx* c, const hkv_exchange* exchange, void* out, void* stream) {
    HKV_CHECK_CTX(c);
    const int stx = check_exchange(c, exchange, "merge_published");
    if (stx) return stx;
    if (!out) return fail(c, HKV_ERR_INVALID_ARG, "merge_published: null output");
    if (!aligned(out, 2)) return fail(c, HKV_ERR_ALIGNMENT, "merge_published: out not 2-byte aligned");
    if (c->g.head_dim > 512) return fail(c, HKV_ERR_GEOMETRY, "merge_published: head_dim above 512");
    MergePublishedArgs a{};
    uint8_t* box = (uint8_t*)exchange->mailbox[exchange->rank];
    for (int r = 0; r < exchange->world; ++r) {
        a.part[r] = (const float*)((const uint8_t*)exchange->mailbox[r] + kMailboxHeaderBytes);
        a.flag_out[r] = (uint32_t*)exchange->mailbox[r] + exchange->rank;
    }
    a.flags = (const uint32_t*)box;
    a.state = (uint32_t*)(box + kMailboxHeaderBytes / 2);
    a.world = exchange->world;
    a.rows = c->g.batch * c->g.num_heads;
    a.HD = c->g.head_dim;
    a.out = (__half*)out;
    a.status = c->d_status;
    a.limit_ns = (unsigned long long)(exchange->wait_limit_ms > 0 ? exchange->wait_limit_ms : 2000) * 1000000ull;
    const unsigned blocks = (unsigned)((a.rows + kMergeWarps - 1) / kMergeWarps);
    hkv_merge_published_kernel<<<blocks, kMergeWarps * 32, 0, (cudaStream_t)stream>>>(a);
    const cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? HKV_OK : fail_cuda(c, e, "merge_published launch");
}

int hkv_prefill_attention(hkv_ctx* c, const void* q, const void* k_cache, const void* v_cache,
                          void* out, int32_t seq_new, int32_t past_len, float scale, void* stream) {
    HKV_CHECK_CTX(c);
    if (!q || !k_cache || !v_cache || !out) return fail(c, HKV_ERR_INVALID_ARG, "prefill: null tensor");
    if (seq_new < 0 || past_len < 0) return fail(c, HKV_ERR_INVALID_ARG, "prefill: negative length");
    if (!aligned(q, 2) || !aligned(k_cache, 2) || !aligned(v_cache, 2) || !aligned(out, 2))
        return fail(c, HKV_ERR_ALIGNMENT, "prefill: fp16 pointer not 2-byte aligned");
    if (c->g.batch != 1) return fail(c, HKV_ERR_GEOMETRY, "prefill: the op is batch 1 (kernels/attention.cu:709)");
    if (!c->workspace) return fail(c, HKV_ERR_WORKSPACE, "prefill: the context was created append-only");
    if (c->g.shard_count > 1) return fail(c, HKV_ERR_GEOMETRY, "prefill: the cache must not be sequence-sharded");
    if (c->g.layout == HKV_LAYOUT_RING) {
        // The ring already holds the chunk. Every position a query attends must still be there: either
        // nothing has been overwritten yet, or the oldest one needed (past_len + 1 - window) lies within
        // `slots` of the newest one written (past_len + seq_new - 1).
        const long long end = (long long)past_len + seq_new;
        const bool fits = end <= c->g.slots ||
                          (c->g.window_size > 0 && (long long)seq_new + c->g.window_size - 1 <= c->g.slots);
        if (!fits)
            return fail(c, HKV_ERR_GEOMETRY, "prefill: chunk + window do not fit the ring (seq_new + window_size - 1 > slots)");
    }
    if (seq_new == 0) return HKV_OK;
    // (the tensor-core kernel takes row maxima before scaling, which needs a positive scale)
    if (prefill_tc_ok(c->g) && scale > 0.0f && aligned(q, 16) && aligned(k_cache, 16) && aligned(v_cache, 16) && aligned(out, 16)) {
        return prefill_tc_launch(c, c->g, q, k_cache, v_cache, out, seq_new, past_len, scale, (cudaStream_t)stream, nullptr);
    }
    PrefillArgs a;
    a.q = (const __half*)q;
    a.k_cache = (const __half*)k_cache;
    a.v_cache = (const __half*)v_cache;
    a.out = (__half*)out;
    a.S_new = seq_new;
    a.past_len = past_len;
    a.H = c->g.num_heads;
    a.KVH = c->g.num_kv_heads;
    a.HD = c->g.head_dim;
    a.slots = c->g.slots;
    a.window = c->g.window_size;
    a.ring = c->g.layout == HKV_LAYOUT_RING ? 1 : 0;
    a.scale_log2 = scale * 1.4426950408889634f;
    dim3 grid((unsigned)seq_new, (unsigned)c->g.num_heads);
    hkv_prefill_generic_kernel<<<grid, kGenWarps * 32, 0, (cudaStream_t)stream>>>(a);
    const cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? HKV_OK : fail_cuda(c, e, "prefill launch");
}

int hkv_prefill_append_attention(hkv_ctx* c, const void* q, const void* k_new, const void* v_new, void* k_cache,
                                 void* v_cache, void* out, int32_t seq_new, int32_t past_len, float scale, void* stream) {
    HKV_CHECK_CTX(c);
    if (!q || !k_new || !v_new || !k_cache || !v_cache || !out) return fail(c, HKV_ERR_INVALID_ARG, "prefill: null tensor");
    if (seq_new < 0 || past_len < 0) return fail(c, HKV_ERR_INVALID_ARG, "prefill: negative length");
    if (c->g.batch != 1) return fail(c, HKV_ERR_GEOMETRY, "prefill: the op is batch 1 (kernels/attention.cu:709)");
    if (seq_new == 0) return HKV_OK;
    const hkv_geometry& g = c->g;
    cudaStream_t st = (cudaStream_t)stream;
    const bool ring = g.layout == HKV_LAYOUT_RING;
    // A plane that holds the chunk next to everything it attends takes the plain order: append, attend.
    const bool plain = !ring ? true
                             : ((long long)past_len + seq_new <= g.slots ||
                                (g.window_size > 0 && (long long)seq_new + g.window_size - 1 <= g.slots));
    if (plain) {
        int stt = launch_append(c, k_new, v_new, k_cache, v_cache, nullptr, 0, past_len, seq_new, st, true);
        if (stt) return stt;
        return hkv_prefill_attention(c, q, k_cache, v_cache, out, seq_new, past_len, scale, stream);
    }
    // Ring too small for that: attend first. Needs the window inside the ring and a partial-row workspace.
    if (g.window_size <= 0 || g.window_size > g.slots || seq_new > g.slots)
        return fail(c, HKV_ERR_GEOMETRY, "prefill: the ring must hold the window (window_size <= slots) and the chunk (seq_new <= slots)");
    if (!prefill_tc_ok(g) || !c->prefill_ws || seq_new > g.max_seq_new || !(scale > 0.0f) || !aligned(q, 16) || !aligned(k_new, 16) ||
        !aligned(v_new, 16) || !aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(out, 16))
        return fail(c, HKV_ERR_GEOMETRY, "prefill: attending before the append needs the tensor-core path (head_dim 64/96/128/256, 16-byte aligned tensors, positive scale) and max_seq_new >= seq_new");
    // pass 1: the rows already in the ring (positions below past_len), partial 0 of 2
    const PrefillPass cached{past_len, 0, 2};
    int stt = prefill_tc_launch(c, g, q, k_cache, v_cache, out, seq_new, past_len, scale, st, &cached);
    if (stt) return stt;
    // pass 2: the chunk's own rows, as a linear plane of seq_new rows with nothing before it: positions
    // are relative to past_len, which leaves the causal and window masks unchanged; partial 1 of 2
    hkv_geometry gc = g;
    gc.slots = seq_new;
    gc.layout = HKV_LAYOUT_LINEAR;
    gc.batch_stride_elems = 0;
    const PrefillPass chunk{0x7fffffff, 1, 2};
    stt = prefill_tc_launch(c, gc, q, k_new, v_new, out, seq_new, 0, scale, st, &chunk);
    if (stt) return stt;
    const long long rows = (long long)seq_new * g.num_heads;
    hkv_prefill_combine_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(c->prefill_ws, (__half*)out, rows, g.num_heads, g.head_dim, 2,
                                                                          kPrefillMaxSplits, nullptr, c->G);
    // and only now the append (it overwrites rows pass 1 has read)
    stt = launch_append(c, k_new, v_new, k_cache, v_cache, nullptr, 0, past_len, seq_new, st, true);
    if (stt) return stt;
    const cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? HKV_OK : fail_cuda(c, e, "prefill launch");
}

int hkv_append_decode_attention_host(hkv_ctx* c, const void* h_q, const void* h_k_new,
                                     const void* h_v_new, void* k_cache, void* v_cache,
                                     void* h_out, const int32_t* d_cache_pos, float scale,
                                     void* stream) {
    HKV_CHECK_CTX(c);
    if (!h_q || !h_k_new || !h_v_new || !h_out) return fail(c, HKV_ERR_INVALID_ARG, "host op: null buffer");
    const size_t qb = (size_t)c->g.batch * c->g.num_heads * c->g.head_dim * 2;
    const size_t kb = (size_t)c->g.batch * c->g.num_kv_heads * c->g.head_dim * 2;
    cudaError_t e;
    if (!c->st_q) {
        if ((e = cudaMalloc(&c->st_q, qb)) != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(staging)");
        if ((e = cudaMalloc(&c->st_k, kb)) != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(staging)");
        if ((e = cudaMalloc(&c->st_v, kb)) != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(staging)");
        if ((e = cudaMalloc(&c->st_out, qb)) != cudaSuccess) return fail_cuda(c, e, "cudaMalloc(staging)");
    }
    cudaStream_t st = (cudaStream_t)stream;
    if ((e = cudaMemcpyAsync(c->st_q, h_q, qb, cudaMemcpyHostToDevice, st)) != cudaSuccess ||
        (e = cudaMemcpyAsync(c->st_k, h_k_new, kb, cudaMemcpyHostToDevice, st)) != cudaSuccess ||
        (e = cudaMemcpyAsync(c->st_v, h_v_new, kb, cudaMemcpyHostToDevice, st)) != cudaSuccess)
        return fail_cuda(c, e, "cudaMemcpyAsync(H2D)");
    if (!d_cache_pos) return fail(c, HKV_ERR_INVALID_ARG, "host op: null position array");
    const int stt = decode_full(c, c->st_q, c->st_k, c->st_v, k_cache, v_cache, c->st_out, nullptr,
                                d_cache_pos, 1, 0, scale, st, nullptr, true);
    if (stt) return stt;
    if ((e = cudaMemcpyAsync(h_out, c->st_out, qb, cudaMemcpyDeviceToHost, st)) != cudaSuccess)
        return fail_cuda(c, e, "cudaMemcpyAsync(D2H)");
    return HKV_OK;
}

int hkv_append_decode_attention_host_pipelined(hkv_ctx* c, const void* h_q, const void* h_k_new,
                                               const void* h_v_new, void* k_cache, void* v_cache,
                                               void* h_out, const int32_t* d_cache_pos, float scale,
                                               void* stream) {
    HKV_CHECK_CTX(c);
    if (!h_q || !h_k_new || !h_v_new || !h_out) return fail(c, HKV_ERR_INVALID_ARG, "host op: null buffer");
    if (!d_cache_pos) return fail(c, HKV_ERR_INVALID_ARG, "host op: null position array");
    const size_t qb = (size_t)c->g.batch * c->g.num_heads * c->g.head_dim * 2;
    const size_t kb = (size_t)c->g.batch * c->g.num_kv_heads * c->g.head_dim * 2;
    cudaError_t e;
    if (!c->host_in) {
        if ((e = cudaStreamCreateWithFlags(&c->host_in, cudaStreamNonBlocking)) != cudaSuccess ||
            (e = cudaStreamCreateWithFlags(&c->host_out, cudaStreamNonBlocking)) != cudaSuccess)
            return fail_cuda(c, e, "cudaStreamCreate(host copies)");
    }
    hkv_ctx::HostSlot& h = c->host_slots[c->host_calls % hkv_ctx::kHostSlots];
    if (!h.q) {
        if ((e = cudaMalloc(&h.q, qb)) != cudaSuccess || (e = cudaMalloc(&h.k, kb)) != cudaSuccess ||
            (e = cudaMalloc(&h.v, kb)) != cudaSuccess || (e = cudaMalloc(&h.out, qb)) != cudaSuccess)
            return fail_cuda(c, e, "cudaMalloc(staging)");
        if ((e = cudaEventCreateWithFlags(&h.in_done, cudaEventDisableTiming)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&h.compute_done, cudaEventDisableTiming)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&h.out_done, cudaEventDisableTiming)) != cudaSuccess)
            return fail_cuda(c, e, "cudaEventCreate(staging)");
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (h.used) {
        // the set's inputs are free once the launch that read them has run; its output once it has been copied out
        if ((e = cudaStreamWaitEvent(c->host_in, h.compute_done, 0)) != cudaSuccess ||
            (e = cudaStreamWaitEvent(st, h.out_done, 0)) != cudaSuccess)
            return fail_cuda(c, e, "cudaStreamWaitEvent(staging reuse)");
    }
    if ((e = cudaMemcpyAsync(h.q, h_q, qb, cudaMemcpyHostToDevice, c->host_in)) != cudaSuccess ||
        (e = cudaMemcpyAsync(h.k, h_k_new, kb, cudaMemcpyHostToDevice, c->host_in)) != cudaSuccess ||
        (e = cudaMemcpyAsync(h.v, h_v_new, kb, cudaMemcpyHostToDevice, c->host_in)) != cudaSuccess ||
        (e = cudaEventRecord(h.in_done, c->host_in)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(st, h.in_done, 0)) != cudaSuccess)
        return fail_cuda(c, e, "cudaMemcpyAsync(H2D)");
    const int stt = decode_full(c, h.q, h.k, h.v, k_cache, v_cache, h.out, nullptr, d_cache_pos, 1, 0, scale, st, nullptr, true);
    if (stt) return stt;
    if ((e = cudaEventRecord(h.compute_done, st)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(c->host_out, h.compute_done, 0)) != cudaSuccess ||
        (e = cudaMemcpyAsync(h_out, h.out, qb, cudaMemcpyDeviceToHost, c->host_out)) != cudaSuccess ||
        (e = cudaEventRecord(h.out_done, c->host_out)) != cudaSuccess)
        return fail_cuda(c, e, "cudaMemcpyAsync(D2H)");
    h.used = true;
    ++c->host_calls;
    return HKV_OK;
}

int hkv_host_flush(hkv_ctx* c, void* stream) {
    HKV_CHECK_CTX(c);
    for (hkv_ctx::HostSlot& h : c->host_slots) {
        if (!h.used) continue;
        const cudaError_t e = cudaStreamWaitEvent((cudaStream_t)stream, h.out_done, 0);
        if (e != cudaSuccess) return fail_cuda(c, e, "cudaStreamWaitEvent(flush)");
    }
    return HKV_OK;
}

int hkv_ctx_profile_begin(hkv_ctx* c, int32_t max_calls) {
    HKV_CHECK_CTX(c);
    if (max_calls < 0 || max_calls > (1 << 20)) return fail(c, HKV_ERR_INVALID_ARG, "profile: bad max_calls");
    while ((int)c->prof_events.size() < max_calls * 3) {
        cudaEvent_t e;
        const cudaError_t err = cudaEventCreate(&e);
        if (err != cudaSuccess) return fail_cuda(c, err, "cudaEventCreate");
        c->prof_events.push_back(e);
    }
    c->prof_calls = 0;
    c->prof_max = max_calls;
    return HKV_OK;
}

int hkv_ctx_profile_end(hkv_ctx* c, void* stream, float* decode_ms, float* combine_ms, int32_t* calls) {
    HKV_CHECK_CTX(c);
    cudaError_t err = cudaStreamSynchronize((cudaStream_t)stream);
    if (err != cudaSuccess) return fail_cuda(c, err, "cudaStreamSynchronize");
    float d = 0.0f, m = 0.0f;
    for (int i = 0; i < c->prof_calls; ++i) {
        float a = 0.0f, b = 0.0f;
        cudaEventElapsedTime(&a, c->prof_events[(size_t)i * 3], c->prof_events[(size_t)i * 3 + 1]);
        cudaEventElapsedTime(&b, c->prof_events[(size_t)i * 3 + 1], c->prof_events[(size_t)i * 3 + 2]);
        d += a;
        m += b;
    }
    if (decode_ms) *decode_ms = d;
    if (combine_ms) *combine_ms = m;
    if (calls) *calls = c->prof_calls;
    c->prof_max = 0;
    c->prof_calls = 0;
    return HKV_OK;
}

int hkv_qk_norm_rope_kv(hkv_ctx* c, void* q, void* k, const void* v, const void* q_norm_w,
                        const void* k_norm_w, void* k_cache, void* v_cache, const int32_t* d_cache_pos,
                        int32_t position, int32_t seq_new, int32_t rotary_dim, float eps, float theta,
                        float scaling_factor, void* stream) {
    HKV_CHECK_CTX(c);
    if (!q || !k || !q_norm_w || !k_norm_w) return fail(c, HKV_ERR_INVALID_ARG, "qk_norm_rope: null tensor");
    if ((k_cache == nullptr) != (v_cache == nullptr) || (k_cache && !v))
        return fail(c, HKV_ERR_INVALID_ARG, "qk_norm_rope: k_cache, v_cache and v go together");
    if (seq_new < 0 || (!d_cache_pos && position < 0)) return fail(c, HKV_ERR_INVALID_ARG, "qk_norm_rope: negative size");
    if (!aligned(q, 2) || !aligned(k, 2) || !aligned(v, 2) || !aligned(k_cache, 2) || !aligned(v_cache, 2) ||
        !aligned(q_norm_w, 2) || !aligned(k_norm_w, 2))
        return fail(c, HKV_ERR_ALIGNMENT, "qk_norm_rope: fp16 pointer not 2-byte aligned");
    if (seq_new == 0) return HKV_OK;
    const hkv_geometry& g = c->g;
    RopeArgs a{};
    a.q = (__half*)q;
    a.k = (__half*)k;
    a.v = (const __half*)v;
    a.q_w = (const __half*)q_norm_w;
    a.k_w = (const __half*)k_norm_w;
    a.k_cache = (__half*)k_cache;
    a.v_cache = (__half*)v_cache;
    a.d_pos = d_cache_pos;
    a.pos_stride = c->pos_stride;
    a.host_pos = position;
    a.map = c->map;
    a.B = g.batch;
    a.S = seq_new;
    a.H = g.num_heads;
    a.KVH = g.num_kv_heads;
    a.HD = g.head_dim;
    // same defaults as the reference launcher (kernels/attention.cu:955-956)
    a.rot = rotary_dim <= 0 ? g.head_dim : (rotary_dim / 2) * 2;
    if (a.rot > g.head_dim) return fail(c, HKV_ERR_INVALID_ARG, "qk_norm_rope: rotary_dim exceeds head_dim");
    a.batch_stride = c->batch_stride;
    a.eps = eps;
    a.theta = theta;
    a.scaling = scaling_factor <= 0.0f ? 1.0f : scaling_factor;
    const long long tokens = (long long)g.batch * seq_new;
    if (a.rot / 2 > 256) return fail(c, HKV_ERR_GEOMETRY, "qk_norm_rope: rotary_dim above 512");
    // register path: 16-byte aligned rows, head_dim and half the rotary span in whole 8-element pieces
    const bool fast = g.head_dim % 8 == 0 && g.head_dim <= 256 && (a.rot / 2) % 8 == 0 && c->batch_stride % 8 == 0 &&
                      aligned(q, 16) && aligned(k, 16) && (!v || aligned(v, 16)) &&
                      (!k_cache || (aligned(k_cache, 16) && aligned(v_cache, 16)));
    const bool copy_v = k_cache && v;
    const int per_tok = g.num_heads + g.num_kv_heads + ((fast ? copy_v : true) ? g.num_kv_heads : 0);
    int heads_per_warp = 1;
    if (fast) {
        int lanes = 1;
        while (lanes < g.head_dim / 8) lanes <<= 1;
        heads_per_warp = 32 / lanes;
    }
    const int warp_units = (per_tok + heads_per_warp - 1) / heads_per_warp;
    // many tokens: a CTA owns a contiguous range of tokens (equal ranges, at most four resident CTAs per
    // SM: one wave); few tokens: one range per token and as many CTAs per token as its units fill, so
    // that a decode launch still spreads over the SMs
    unsigned gx = 1, gy;
    if (tokens >= 2LL * c->sm_count) {
        const long long per = (tokens + 4LL * c->sm_count - 1) / (4LL * c->sm_count);
        gy = (unsigned)((tokens + per - 1) / per);
    } else {
        gx = (unsigned)((warp_units + kRopeWarps - 1) / kRopeWarps);
        gy = (unsigned)tokens;
    }
    hkv_qk_norm_rope_kernel<<<dim3(gx, gy), kRopeWarps * 32, 0, (cudaStream_t)stream>>>(a, fast ? 1 : 0);
    const cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? HKV_OK : fail_cuda(c, e, "qk_norm_rope launch");
}

int hkv_ctx_selftest_bounded_wait(hkv_ctx* c, int32_t limit_ms, void* stream) {
    HKV_CHECK_CTX(c);
    if (limit_ms <= 0 || limit_ms > 1000) return fail(c, HKV_ERR_INVALID_ARG, "selftest: limit must be 1..1000 ms");
    hkv_selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c->d_status, (unsigned long long)limit_ms * 1000000ull,
                                                                nullptr);
    const cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? HKV_OK : fail_cuda(c, e, "selftest launch");
}

int32_t hkv_slot_of_position(const hkv_geometry* g, int32_t pos) {
    const char* why;
    if (validate_geometry(g, &why) != HKV_OK) return -1;
    return slot_of_pos(make_map(*g), pos);
}

int32_t hkv_position_of_slot(const hkv_geometry* g, int32_t slot, int32_t total_seq) {
    const char* why;
    if (validate_geometry(g, &why) != HKV_OK || slot < 0 || slot >= g->slots) return -1;
    return pos_of_slot(make_map(*g), slot, total_seq);
}

int hkv_plan_sequence(const hkv_geometry* g, int32_t total_seq, int32_t chunk_tiles,
                      int32_t* first, int32_t* tile_lo, int32_t* n_tiles, int32_t* n_chunks) {
    const char* why;
    const int st = validate_geometry(g, &why);
    if (st) return st;
    if (chunk_tiles <= 0 || total_seq < 0) return HKV_ERR_INVALID_ARG;
    const SeqMap m = make_map(*g);
    int tl, nt;
    tile_range(m, total_seq, tl, nt);
    if (first) *first = first_pos(m, total_seq);
    if (tile_lo) *tile_lo = tl;
    if (n_tiles) *n_tiles = nt;
    if (n_chunks) *n_chunks = (nt + chunk_tiles - 1) / chunk_tiles;
    return HKV_OK;
}

int hkv_plan_decode_tiles(const hkv_geometry* g, int32_t total_seq, int32_t* tile_lo, int32_t* n_tiles, int32_t* wrap_tiles) {
    const char* why;
    const int st = validate_geometry(g, &why);
    if (st) return st;
    if (total_seq < 0) return HKV_ERR_INVALID_ARG;
    const SeqMap m = make_map(*g);
    int tl = 0, nt = 0, wt = 0;
    if (tma_stale_ring(*g)) {
        tma_tile_range(m, total_seq, tl, nt, wt);
        if (wt == 0x7fffffff) wt = 0;
    } else {
        tile_range(m, total_seq, tl, nt);
    }
    if (tile_lo) *tile_lo = tl;
    if (n_tiles) *n_tiles = nt;
    if (wrap_tiles) *wrap_tiles = wt;
    return HKV_OK;
}

int hkv_plan_decode_spans(const hkv_geometry* g, const int32_t* totals, int32_t spans_wanted, int32_t* first_span,
                          int32_t* n_parts, int32_t* total_tiles, int32_t* spans_used) {
    const char* why;
    const int st = validate_geometry(g, &why);
    if (st) return st;
    if (!totals || spans_wanted <= 0) return HKV_ERR_INVALID_ARG;
    const SeqMap m = make_map(*g);
    const bool stale = tma_stale_ring(*g);
    // the same tile table the decode kernel builds in shared memory and leaves for the merge kernel
    std::vector<int> pre((size_t)g->batch + 1, 0);
    for (int b = 0; b < g->batch; ++b) {
        int tl = 0, nt = 0, wt = 0;
        if (stale) tma_tile_range(m, totals[b], tl, nt, wt);
        else tile_range(m, totals[b], tl, nt);
        pre[(size_t)b + 1] = pre[(size_t)b] + nt;
    }
    const int W = pre[(size_t)g->batch];
    const int spans = span_count(W, spans_wanted);
    for (int b = 0; b < g->batch; ++b) {   // what hkv_combine_*_kernel derives for sequence b
        const int p0 = pre[(size_t)b], p1 = pre[(size_t)b + 1];
        const int first = p1 > p0 ? span_owner(p0, W, spans) : 0;
        if (first_span) first_span[b] = first;
        if (n_parts) n_parts[b] = p1 > p0 ? span_owner(p1 - 1, W, spans) - first + 1 : 0;
    }
    if (total_tiles) *total_tiles = W;
    if (spans_used) *spans_used = spans;
    return HKV_OK;
}

int hkv_plan_prefill(const hkv_geometry* g, int32_t seq_new, int32_t past_len, int32_t sm_count,
                     int32_t* tiles_in_flight, int32_t* items, int32_t* splits, int32_t* min_span_tiles) {
    const char* why;
    const int st = validate_geometry(g, &why);
    if (st) return st;
    if (seq_new <= 0 || past_len < 0 || sm_count <= 0) return HKV_ERR_INVALID_ARG;
    if (!prefill_tc_ok(*g)) {   // the SIMT kernel: one CTA per (query, head), no split
        if (tiles_in_flight) *tiles_in_flight = 0;
        if (items) *items = seq_new * g->num_heads;
        if (splits) *splits = 1;
        if (min_span_tiles) *min_span_tiles = 0;
        return HKV_OK;
    }
    PrefillTcArgs t{};
    t.key_limit = 0x7fffffff;
    int pair = 0, min_span = 0, grid = 0, max_parts = 0;
    std::vector<double> scratch;
    plan_prefill_tc(*g, seq_new, past_len, sm_count, g->max_seq_new >= seq_new, t, pair, min_span, grid, max_parts, scratch);
    if (tiles_in_flight) *tiles_in_flight = pair ? 2 : 1;
    if (items) *items = t.streamk ? grid : t.n_qtiles * t.KVH * t.splits;
    if (splits) *splits = t.streamk ? 0 : t.splits;
    if (min_span_tiles) *min_span_tiles = min_span;
    return HKV_OK;
}

int32_t hkv_preferred_prefill_chunk(const hkv_geometry* g, int32_t sm_count, int32_t target) {
    const char* why;
    if (validate_geometry(g, &why) || sm_count <= 0 || target <= 0) return -1;
    if (!prefill_tc_ok(*g)) return target;
    const int G = g->num_heads / g->num_kv_heads;
    const int q_pair = (g->head_dim == 256 ? 1 : 2) * (kPfRows / G);   // queries per work item
    int a = sm_count, b = g->num_kv_heads;
    while (b) { const int r = a % b; a = b; b = r; }   // a = gcd
    const long long unit = (long long)(sm_count / a) * q_pair;   // queries per whole round of items
    const long long k = target / unit;
    const long long best = (k > 0 ? k : 1) * unit;
    return best > 0x7fffffffLL ? target : (int32_t)best;
}

int hkv_fill_synthetic(void* dst, uint64_t seed, uint64_t first_index, uint64_t count, void* stream) {
    if (!dst && count) return HKV_ERR_INVALID_ARG;
    if (!aligned(dst, 2)) return HKV_ERR_ALIGNMENT;
    if (count == 0) return HKV_OK;
    unsigned long long blocks = (count + 255) / 256;
    if (blocks > 148ull * 32) blocks = 148ull * 32;
    hkv_fill_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((__half*)dst, seed, first_index,
                                                                        count);
    return cudaPeekAtLastError() == cudaSuccess ? HKV_OK : HKV_ERR_CUDA;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate
// ---------------------------------------------------------------------------
// Some hosts of this library cannot call cudaMalloc at the point where they need
// attention: code running under a memory plan fixed at start-up (every byte of HBM already
// handed to the KV planes), plugin sandboxes that forbid allocation after initialisation,
// and latency-critical serving threads for which an allocation's implicit device
// synchronisation is not acceptable. hkv_decode_attention_static serves them: the split-K
// partials live in the fixed array below instead of a context-owned workspace.
//
// The array is part of the library image, so EVERY GPU that loads libhkv holds these
// HKV_STATIC_SCRATCH_BYTES (8 MiB) from load until the process exits, used or not.
//
// In host code the name `g_static_scratch` is only a host-side stand-in for the symbol, not
// a device address; the address a kernel may use comes from cudaGetSymbolAddress, asked
// once per device with that device current (static_scratch_for_current_device below).
static __device__ __align__(256) unsigned char g_static_scratch[HKV_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kStaticMaxDevices = 64;
struct StaticDeviceSlot {
    void* scratch = nullptr;  // device address of g_static_scratch on this device
    int sm_count = 0;
};
StaticDeviceSlot g_static_slots[kStaticMaxDevices];
std::mutex g_static_mutex;

// Set-up, once per device: resolves the device address of the array on the CURRENT device.
// Runs on the first call made on that device; no allocation, but the runtime may load the
// module here, so that first call belongs before any stream capture.
int static_scratch_for_current_device(StaticDeviceSlot* out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return HKV_ERR_NO_DEVICE;
    }
    if (dev < 0 || dev >= kStaticMaxDevices) return HKV_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticDeviceSlot& slot = g_static_slots[dev];
    if (!slot.scratch) {
        int major = 0, sm = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
            cudaGetLastError();
            return HKV_ERR_CUDA;
        }
        if (major != 10) return HKV_ERR_NO_DEVICE;
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return HKV_ERR_CUDA;
        }
        slot.sm_count = sm;
        slot.scratch = p;
    }
    *out = slot;
    return HKV_OK;
}

}  // namespace

extern "C" int hkv_decode_attention_static(const hkv_geometry* geometry, const void* q,
                                           const void* k_cache, const void* v_cache, void* out,
                                           const int32_t* d_total_seq, float scale, void* stream) {
    const char* why = "";
    const int vst = validate_geometry(geometry, &why);
    if (vst) return vst;
    if (!q || !k_cache || !v_cache || !out || !d_total_seq) return HKV_ERR_INVALID_ARG;
    if (!aligned(q, 2) || !aligned(k_cache, 2) || !aligned(v_cache, 2) || !aligned(out, 2))
        return HKV_ERR_ALIGNMENT;
    if (!std::isfinite(scale)) return HKV_ERR_INVALID_ARG;
    StaticDeviceSlot slot;
    const int sst = static_scratch_for_current_device(&slot);
    if (sst) return sst;

    // Split plan: the caller's chunk size (or the automatic one), coarsened until the
    // partials fit the fixed array; refuse if even one partial per (sequence, head) does not.
    const hkv_geometry& g = *geometry;
    int chunk_tiles, max_chunks;
    fill_plan(g, slot.sm_count, chunk_tiles, max_chunks);
    const int tiles = (g.slots + kTileRows - 1) / kTileRows;
    while (workspace_bytes_for(g, max_chunks) > (size_t)HKV_STATIC_SCRATCH_BYTES && max_chunks > 1) {
        chunk_tiles *= 2;
        max_chunks = (tiles + chunk_tiles - 1) / chunk_tiles;
    }
    if (workspace_bytes_for(g, max_chunks) > (size_t)HKV_STATIC_SCRATCH_BYTES)
        return HKV_ERR_TOO_LARGE;  // batch * num_heads * (head_dim + 2) * 4 bytes exceeds the array

    // Nothing in the array has to start at zero: the combine kernel reads exactly the partial
    // rows the decode kernel of the same call has written (both derive the count from
    // d_total_seq), so the previous call's contents are never observed.
    DecodeArgs a{};
    a.q = (const __half*)q;
    a.k_cache = (const __half*)k_cache;
    a.v_cache = (const __half*)v_cache;
    a.k_new = nullptr;
    a.v_new = nullptr;
    a.k_cache_w = nullptr;
    a.v_cache_w = nullptr;
    a.part = static_cast<float*>(slot.scratch);
    a.span_part = nullptr;
    a.gpre = nullptr;
    a.span_gang = 1;
    a.total = d_total_seq;
    a.status = nullptr;  // the SIMT kernel has no waits and never touches the status word
    a.map = make_map(g);
    a.B = g.batch;
    a.H = g.num_heads;
    a.KVH = g.num_kv_heads;
    a.HD = g.head_dim;
    a.chunk_tiles = chunk_tiles;
    a.max_chunks = max_chunks;
    a.pos_is_index = 0;
    a.pos_stride = (g.flags & HKV_FLAG_SCALAR_POSITION) ? 0 : 1;
    a.host_len = 0;
    a.batch_stride = g.batch_stride_elems ? g.batch_stride_elems
                                          : (long long)g.slots * g.num_kv_heads * g.head_dim;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.q_stride = g.q_seq_stride_elems ? g.q_seq_stride_elems : (long long)g.num_heads * g.head_dim;
    a.new_stride = (long long)g.num_kv_heads * g.head_dim;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((unsigned)max_chunks, (unsigned)g.num_heads, (unsigned)g.batch);
    hkv_decode_generic_kernel<<<grid, kGenWarps * 32, 0, st>>>(a);

    CombineArgs c{};
    const long long PW = g.head_dim + 2;
    c.part = static_cast<const float*>(slot.scratch);
    c.stride_b = (long long)max_chunks * g.num_heads * PW;
    c.stride_c = (long long)g.num_heads * PW;
    c.total = d_total_seq;
    c.pos_is_index = 0;
    c.pos_stride = a.pos_stride;
    c.host_len = 0;
    c.fixed_count = 0;
    c.gpre = nullptr;
    c.span_spans = 0;
    c.B = g.batch;
    c.map = a.map;
    c.chunk_tiles = chunk_tiles;
    c.H = g.num_heads;
    c.HD = g.head_dim;
    c.out = (__half*)out;
    c.out_partial = nullptr;
    hkv_combine_kernel<<<dim3((unsigned)g.num_heads, (unsigned)g.batch), kCombineThreads, 0, st>>>(c);
    return cudaPeekAtLastError() == cudaSuccess ? HKV_OK : HKV_ERR_CUDA;
}
