// hkv_common.cuh — shared device-side definitions: how a sequence's logical positions
// map to rows ("slots") of a cache plane, how a sequence is cut into split-K work
// items, the partial (m, l, o) format, and thin wrappers over the sm_100a PTX used by
// the kernels (mbarrier, bulk-tensor copies, ldmatrix, mma, movmatrix).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hkv {

constexpr int kTileRows = 64;          // rows per split-K tile (unit of chunk_tiles)
constexpr float kNegBig = -1.0e30f;    // "minus infinity" that survives subtraction
constexpr int kStatusWaitRanOut = 1;   // device status bits
constexpr int kStatusBoundCheck = 2;
constexpr int kMaxPeers = 8;           // ranks of one node in a peer exchange (HKV_MAX_PEERS)

// How logical positions of one sequence map to rows of its cache plane.
struct SeqMap {
    int slots;        // rows per sequence
    int layout;       // 0 linear, 1 ring
    int window;       // 0 = none
    int shard_rank;   // block-cyclic sequence split (shard_count <= 1: off)
    int shard_count;
    int shard_block;
};

// Row that holds logical position p on this rank, or -1 (not stored here / dropped).
__host__ __device__ inline int slot_of_pos(const SeqMap& m, int p) {
    if (p < 0) return -1;
    if (m.shard_count > 1) {
        const int blk = p / m.shard_block;
        if (blk % m.shard_count != m.shard_rank) return -1;
        const int s = (blk / m.shard_count) * m.shard_block + p % m.shard_block;
        return s < m.slots ? s : -1;
    }
    if (m.layout == 1) return p % m.slots;
    return p < m.slots ? p : -1;  // reference drops rows past the plane (attention.cu:1143)
}

// Logical position held by row s when the sequence has `total` positions; may be < 0
// or >= total (then the row is not attended).
__host__ __device__ inline int pos_of_slot(const SeqMap& m, int s, int total) {
    if (m.shard_count > 1) {
        return ((s / m.shard_block) * m.shard_count + m.shard_rank) * m.shard_block +
               s % m.shard_block;
    }
    if (m.layout == 1) {
        const int last = total - 1;
        int r = (last - s) % m.slots;
        if (r < 0) r += m.slots;
        return last - r;
    }
    return s;
}

// First attended logical position (reference: kernels/attention.cu:385-389).
__host__ __device__ inline int first_pos(const SeqMap& m, int total) {
    int f = m.window > 0 ? (total - m.window > 0 ? total - m.window : 0) : 0;
    if (m.layout == 1 && total - m.slots > f) f = total - m.slots;
    return f;
}

// Rows [lo, hi) of this rank's plane that can hold attended positions.
__host__ __device__ inline void slot_range(const SeqMap& m, int total, int& lo, int& hi) {
    if (total <= 0) { lo = hi = 0; return; }
    if (m.shard_count > 1) {
        const int full = total / m.shard_block, rem = total % m.shard_block;
        int n = ((full + m.shard_count - 1 - m.shard_rank) / m.shard_count) * m.shard_block;
        if (full % m.shard_count == m.shard_rank) n += rem;
        lo = 0;
        hi = n < m.slots ? n : m.slots;
        return;
    }
    if (m.layout == 1 && total > m.slots) { lo = 0; hi = m.slots; return; }
    lo = first_pos(m, total);
    hi = total < m.slots ? total : m.slots;
    if (lo > hi) lo = hi;
}

// Split-K work items of one sequence: tiles are kTileRows-aligned in row space.
__host__ __device__ inline void tile_range(const SeqMap& m, int total, int& tile_lo, int& n_tiles) {
    int lo, hi;
    slot_range(m, total, lo, hi);
    if (hi <= lo) { tile_lo = 0; n_tiles = 0; return; }
    tile_lo = lo / kTileRows;
    n_tiles = (hi + kTileRows - 1) / kTileRows - tile_lo;
}
// Tiles of one sequence for the TMA decode kernel: as tile_range(), except that a wrapped ring LARGER than its window
// (a plane sized for chunked prefill: window + chunk - 1 rows) contributes only the tiles its window touches — a
// cyclic run of tiles starting at the window's first row — instead of the whole ring. `wrap_tiles` is the ring's
// tile count when the run is cyclic (tile index tile_lo + t wraps there), else a number no index reaches.
__host__ __device__ inline void tma_tile_range(const SeqMap& m, int total, int& tile_lo, int& n_tiles, int& wrap_tiles) {
    wrap_tiles = 0x7fffffff;
    if (m.layout == 1 && m.shard_count <= 1 && total > m.slots && m.window > 0 && m.window < m.slots &&
        m.slots % kTileRows == 0) {
        const int ring_tiles = m.slots / kTileRows;
        const int s_first = (total - m.window) % m.slots;
        const int n = (s_first % kTileRows + m.window + kTileRows - 1) / kTileRows;
        tile_lo = s_first / kTileRows;
        n_tiles = n < ring_tiles ? n : ring_tiles;
        wrap_tiles = ring_tiles;
        return;
    }
    tile_range(m, total, tile_lo, n_tiles);
}

__host__ __device__ inline int num_chunks(const SeqMap& m, int total, int chunk_tiles) {
    int tile_lo, n_tiles;
    tile_range(m, total, tile_lo, n_tiles);
    return (n_tiles + chunk_tiles - 1) / chunk_tiles;
}

// Equal-span schedule of the TMA decode kernel: the W tiles of a launch form one line that is cut
// into `spans` equal contiguous pieces with boundaries floor(W * c / spans). Never more spans than
// tiles, so that no span is empty.
__host__ __device__ inline int span_count(int W, int spans_wanted) { return W < spans_wanted ? W : spans_wanted; }
// The span that owns tile x: the largest c whose boundary is <= x.
__host__ __device__ inline int span_owner(long long x, long long W, int spans) {
    return (int)(((x + 1) * spans + W - 1) / W - 1);
}

// Arguments shared by the decode kernels.
struct DecodeArgs {
    const __half* q;        // [B, H, HD]
    const __half* k_cache;  // [B, slots, KVH, HD]
    const __half* v_cache;
    const __half* k_new;    // fused append: [B, KVH, HD] or null
    const __half* v_new;
    __half* k_cache_w;      // writable aliases of the planes (fused append)
    __half* v_cache_w;
    float* part;            // [B, max_chunks, H, HD+2]: o[HD], m (log2 domain), l (chunked schedule)
    float* span_part;       // [spans + B, H, HD+2]: the same rows under the equal-span schedule, the
                            //   piece of sequence b inside span s at slot s + b
    int* gpre;              // [B+1] tiles before each sequence, written by the kernel for the merge
    int span_gang;          // CTAs sharing a span, CTA m of the gang taking the kv heads m, m + gang, ...
    const int32_t* total;   // [B] attended length, or cache position when pos_is_index; null -> host_len
    int32_t* status;        // device status word
    SeqMap map;
    int B, H, KVH, HD;
    int chunk_tiles, max_chunks;
    int pos_is_index;       // 1: total[b] holds cache_pos, attended length = cache_pos + 1
    int pos_stride;         // 1: one position per sequence; 0: every sequence reads total[0]
                            //    (the reference's scalar, kernels/attention.cu:351)
    int host_len;           // attended length of every sequence when total is null
    long long batch_stride; // elements
    float scale_log2;       // scale * log2(e)
    long long q_stride;     // elements between sequences' q rows (H*HD when dense)
    long long new_stride;   // elements between sequences' k_new / v_new rows (KVH*HD when dense)
};

// Attended length of sequence b from a device position array (one entry per sequence, or one
// shared entry when pos_stride == 0) or, when the array is null, from a value passed by the host.
__device__ __forceinline__ int length_of(const int32_t* total, int pos_stride, int pos_is_index,
                                         int host_len, int b) {
    const int t = total ? total[b * pos_stride] + pos_is_index : host_len;
    return t > 0 ? t : 0;
}
__device__ __forceinline__ int attended_len(const DecodeArgs& a, int b) {
    return length_of(a.total, a.pos_stride, a.pos_is_index, a.host_len, b);
}

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit_ns` (2 s by default) of wall time, records it in the status word and
// returns false so the caller can leave its loops; the context stays usable.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int32_t* status,
                                          unsigned long long limit_ns = 2000000000ull) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        for (int i = 0; i < 1024; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > limit_ns) break;
    }
    atomicOr(status, kStatusWaitRanOut);
    return false;
}

// One lane of a converged warp, chosen by the hardware. Unlike `lane == 0` this tells the compiler
// that the guarded code is executed by a single thread of a converged warp, so descriptors and
// addresses of the issue loops can live in uniform registers instead of being moved there per
// instruction.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "@p mov.s32 %0, 1;\n\t}"
        : "+r"(pred));
    return pred != 0;
}

// 4-D bulk-tensor load global -> shared (no multicast), completion on an mbarrier.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace hkv
