// hkv_prefill_tc.cuh — attention of a chunk of new queries over the cache on the 5th-gen
// tensor cores (tcgen05.mma, accumulators in tensor memory), batch 1.
//
// Replaces attention_prefill_cached_kernel (reference kernels/attention.cu:664-788), which
// runs one CTA per (query, head) and re-reads the K/V rows once per query and per head of a
// group. Semantics kept: query i attends cache rows [first_i, past_len + i] with
// first_i = window > 0 ? max(0, past_len + i + 1 - window) : 0.
//
// Shape of the computation
//   * Work item = (tile of QT queries, KV head). The G query heads of the KV head are stacked
//     into the M dimension: row r of the 128-row tile is (query r / G, head r % G), QT = 128 / G
//     queries per tile (18 for a group of 7: 126 of 128 rows used). One bulk-tensor load with
//     box {64 halfs, G heads, QT queries} brings the tile in as 128-byte-swizzled K-major rows.
//   * Warp 8 (one lane) is the TMA producer: Q tile per item; K tiles of 128 (64) cache rows through
//     a 2-stage ring and V tiles through a 3 (2)-stage ring (full/empty mbarriers each).
//   * Warp 9 (one lane) issues the MMAs:  S = Q·K^T  (M128 x N128 x K=HD, both operands K-major
//     from shared memory) into one of two S buffers in tensor memory, and
//     PV = P·V  (A = P from tensor memory as packed fp16, B = V straight from its row-major
//     tile as an MN-major operand). S of tile t+1 is issued before PV of tile t, so the score
//     contraction overlaps the softmax of the previous tile.
//   * Warps 0-7: two threads per row (each half of the score columns and of the output
//     dimensions). The row's scores are read once from tensor memory, masked (causal +
//     window), the two halves exchange their maxima through shared memory, exp2 / sum, and P
//     goes back to tensor memory as packed fp16 (tcgen05.st, two P buffers). O accumulates in
//     tensor memory across the whole item; it is rescaled in place only when a row's maximum
//     outgrows its reference by more than 2^8, so the softmax of tile t+1 overlaps P·V of tile t.
//   * All waits are bounded mbarrier waits; a wait that runs out sets the status word, the
//     roles leave their loops, outstanding copies are drained and tensor memory is freed.
//   * head_dim 64, 96, 128 and 256 (96 staged as 128 with zero-filled columns; 256 with 64-row K/V
//     tiles); linear planes and ring planes (position p in row p % slots) alike: tiles are counted in
//     logical positions and only the row coordinate of a tile's loads wraps.
#pragma once

#include <cuda.h>

#include "hkv_common.cuh"

namespace hkv {

struct PrefillTcArgs {
    __half* out;      // [S_new, H, HD]
    int32_t* status;
    int S_new, past_len, H, KVH, G, QT, n_qtiles, slots, window;
    int HD;           // the tensors' real head_dim (96 is staged as 128 with zero-filled columns)
    int ring;         // 1: ring plane, position p lives in row p % slots (slots % tile rows == 0)
    float scale_log2;
    // Key-range split: every (query tile, kv head) is cut into `splits` consecutive key ranges
    // so that the work items fill the last wave of SMs; with splits > 1 each range writes an
    // un-normalised partial row (o[HD], reference maximum, sum) to `part`
    // [S_new][splits][H][HD+2] and the combine kernel merges them.
    int splits;
    float* part;
    int* item_counter;   // two-tile kernel: zeroed before the launch; items beyond the first of each CTA come from it
    // Equal-span schedule of the two-tile kernel: items are cut where the spans fall, so the number of
    // partial rows differs from row to row; each (query, kv head) records its count in row_parts and
    // partial p of query q sits at part[(q * part_stride + p) ...].
    // Attend-before-append (a plane that cannot hold the chunk next to what it attends): the chunk is
    // attended in two passes — the rows already cached (keys below key_limit = past_len) and the chunk's
    // own rows (a second launch over k_new/v_new as a plane of their own) — each writing partial
    // out_part of out_parts for every row, whatever its own splits.
    int key_limit;       // attend keys below this position only; INT_MAX = no limit
    int out_part;        // with out_parts > 0: the partial slot every row of this launch writes
    int out_parts;       // 0 = decided by the schedule
    int streamk;
    int sk_whole;        // items (longest first) run whole before the equal spans; a multiple of the grid
    int sk_grid;         // CTAs that share the remaining items' key tiles
    int part_stride;
    int* row_parts;      // [S_new][KVH] or null
};

constexpr int kPfRows = 128;   // M of the MMA = rows of a query tile
constexpr int kPfKeys = 128;   // cache rows per K/V tile = N of the score MMA
constexpr int kPfThreads = 320;  // 8 softmax warps + TMA producer + MMA issuer

// K tiles in flight (freed right after the score MMA) and V tiles in flight (freed after the output
// MMA) of the one-tile kernel; head_dim 256 has room for two of each only.
__host__ __device__ constexpr int prefill_tc_k_stages(int) { return 2; }
__host__ __device__ constexpr int prefill_tc_v_stages(int HD) { return HD == 256 ? 2 : 3; }
// Staged head dimension and cache rows per K/V tile for a real head_dim.
__host__ __device__ constexpr int prefill_tc_staged_hd(int head_dim) { return head_dim == 96 ? 128 : head_dim; }
__host__ __device__ constexpr int prefill_tc_keys(int head_dim) { return head_dim == 256 ? 64 : 128; }

__host__ __device__ constexpr size_t prefill_tc_smem_bytes(int HD /*staged*/) {
    return 1024 + (size_t)kPfRows * HD * 2 +
           (size_t)(prefill_tc_k_stages(HD) + prefill_tc_v_stages(HD)) * prefill_tc_keys(HD) * HD * 2 + 40 * 8 + 6 * kPfRows * 4;
}

// ---- geometry of a work item, shared by the kernels and the host planner ----------------------
// Tiles count `keys` LOGICAL positions; in a linear plane a position is its row, in a ring plane
// position p lives in row p % slots (a tile never straddles the wrap: slots % keys == 0).
__host__ __device__ inline int prefill_tile_row(const PrefillTcArgs& a, int pos0) { return a.ring ? pos0 % a.slots : pos0; }
// Positions [0, kv_valid) hold data; beyond them a plane may hold stale bits.
__host__ __device__ inline int prefill_kv_valid(const PrefillTcArgs& a) {
    const int end = a.past_len + a.S_new;
    const int v = (a.ring || end < a.slots) ? end : a.slots;
    return v < a.key_limit ? v : a.key_limit;
}
// Last key a query at position qpos may attend (a linear plane drops rows past its end; a pass
// limited to the rows already cached stops below key_limit).
__host__ __device__ inline int prefill_last_key(const PrefillTcArgs& a, int qpos) {
    const int k = (a.ring || qpos < a.slots) ? qpos : a.slots - 1;
    return k < a.key_limit ? k : a.key_limit - 1;
}
// Key tiles an item of `q_item` queries (item index qt) spans, before any key split.
__host__ __device__ inline void prefill_item_tiles(const PrefillTcArgs& a, int q_item, int keys, int qt, int& kt0, int& ntot) {
    const int q0 = qt * q_item;
    const int first_min = a.window > 0 ? (a.past_len + q0 + 1 - a.window > 0 ? a.past_len + q0 + 1 - a.window : 0) : 0;
    const int q_last = q0 + q_item < a.S_new ? q0 + q_item : a.S_new;
    const int last_max = prefill_last_key(a, a.past_len + q_last - 1);
    kt0 = first_min / keys;
    ntot = last_max / keys - kt0 + 1;
    if (ntot < 1) ntot = 1;
}
// This split's share of the span (the host guarantees splits <= shortest span).
__host__ __device__ inline void prefill_tile_span(const PrefillTcArgs& a, int q_item, int keys, int qt, int sp, int& kt_lo, int& nt) {
    int kt0, ntot;
    prefill_item_tiles(a, q_item, keys, qt, kt0, ntot);
    const int base = ntot / a.splits, rem = ntot % a.splits;
    kt_lo = kt0 + sp * base + (sp < rem ? sp : rem);
    nt = base + (sp < rem ? 1 : 0);
}

// ---- tcgen05 wrappers -------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Tensor-memory row access for the calling thread's lane: 32 consecutive 32-bit columns in,
// 16 consecutive columns out. volatile + memory clobber: the same address is re-read after
// the tensor core has rewritten it, so these must never be merged or hoisted.
__device__ __forceinline__ void tmem_ld32(uint32_t (&v)[32], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 :
                 : "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 :
                 : "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart.
// K-major operands ignore the leading-dimension offset; MN-major operands use it as the
// distance between 64-element column blocks.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((1024u >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version for sm_100
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// ---- softmax arithmetic: the softmax warps are issue-bound, so every element costs as few
// instructions as sm_100 allows: 3-input max, packed two-lane fp32 FMA/ADD, bare ex2.approx.
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// (d0, d1) = (a0, a1) * (b, b) + (c, c)
__device__ __forceinline__ void ffma2_bcast(float& d0, float& d1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// (d0, d1) += (a0, a1)
__device__ __forceinline__ void fadd2_acc(float& d0, float& d1, float a0, float a1) {
    asm("{\n\t.reg .b64 ra, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\t"
        "add.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1)
        : "f"(a0), "f"(a1));
}

// Rare path of the softmax warps: scale this thread's n32*32 columns of O (tensor memory) by
// alpha. Kept out of line so that its registers do not weigh on the per-tile loop.
__device__ __noinline__ void tmem_scale_columns(uint32_t addr, int n32, float alpha) {
    for (int c = 0; c < n32; ++c) {
        uint32_t v[32];
        tmem_ld32(v, addr + c * 32);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
        tmem_st32(addr + c * 32, v);
    }
    tc_wait_st();
}

// HD is the head dimension the tiles are staged with — 64, 128 or 256; head_dim 96 runs as
// HD = 128 with the columns 96..127 of Q, K and V zero-filled by the bulk-tensor loads (they lie
// outside the tensors), which changes neither Q·K^T nor the first 96 columns of P·V. KEYS is the
// number of cache rows per K/V tile: 128, or 64 for head_dim 256, where shared memory (a 64 KB
// query tile) and tensor memory (256 output columns) leave room for half-height tiles only.
template <int HD, int KEYS>
__global__ void __launch_bounds__(kPfThreads, 1)
hkv_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const PrefillTcArgs a) {
    static_assert(HD == 64 || HD == 128 || HD == 256, "staged head_dim 64, 128 or 256");
    static_assert(KEYS == 64 || KEYS == 128, "64 or 128 cache rows per tile");
    static_assert(3 * KEYS + HD <= 512, "tensor-memory columns");
    constexpr int NCH = HD / 64;                       // 64-half column blocks
    constexpr int Q_CHUNK = kPfRows * 128;             // one column block of the 128-row query tile
    constexpr int KV_CHUNK = KEYS * 128;               // one column block of a K/V tile
    constexpr int Q_TILE = kPfRows * HD * 2;
    constexpr int KV_TILE = KEYS * HD * 2;
    constexpr int KST = prefill_tc_k_stages(HD), VST = prefill_tc_v_stages(HD);
    constexpr int KH = KEYS / 2;                       // score columns per softmax thread
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t COL_S0 = 0, COL_S1 = KEYS, COL_PV = 2 * KEYS, COL_P0 = 2 * KEYS + HD, COL_P1 = COL_P0 + KEYS / 2;
    constexpr uint32_t IDESC_QK = (1u << 4) | ((uint32_t)(KEYS >> 3) << 17) | ((uint32_t)(kPfRows >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(kPfRows >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_gen = smem;                                   // Q tile
    uint8_t* k_gen = smem + Q_TILE;                          // KST K tiles
    uint8_t* v_gen = k_gen + KST * KV_TILE;                  // VST V tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_gen + VST * KV_TILE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
    float* xch = reinterpret_cast<float*>(bars + 40);   // [2 buffers][2 halves][128] maxima + [2][128] sums
    const uint32_t q_smem = smem_u32(q_gen), k_smem = smem_u32(k_gen), v_smem = smem_u32(v_gen);
    const uint32_t bar0 = smem_u32(bars);
    // barrier map (8 bytes each)
    const uint32_t B_QFULL = bar0, B_QEMPTY = bar0 + 8;
    const uint32_t B_KFULL = bar0 + 16;     // [2]
    const uint32_t B_KEMPTY = bar0 + 32;    // [2]
    const uint32_t B_VFULL = bar0 + 48;     // [3]
    const uint32_t B_VEMPTY = bar0 + 72;    // [3]
    const uint32_t B_SFULL = bar0 + 96;     // [2]
    const uint32_t B_SFREE = bar0 + 112;    // [2]
    const uint32_t B_PFULL = bar0 + 128, B_PVFULL = bar0 + 136, B_DONE = bar0 + 144;
    const uint32_t B_XCH = bar0 + 152;      // softmax threads exchanging row maxima / sums
    const uint32_t B_OFULL = bar0 + 160;    // last P·V of an item has completed

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(B_QFULL, 1); mbar_init(B_QEMPTY, 1);
        for (int s = 0; s < KST; ++s) { mbar_init(B_KFULL + 8 * s, 1); mbar_init(B_KEMPTY + 8 * s, 1); }
        for (int s = 0; s < VST; ++s) { mbar_init(B_VFULL + 8 * s, 1); mbar_init(B_VEMPTY + 8 * s, 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(B_SFULL + 8 * s, 1); mbar_init(B_SFREE + 8 * s, 256); }
        mbar_init(B_PFULL, 256); mbar_init(B_PVFULL, 1); mbar_init(B_DONE, 1); mbar_init(B_XCH, 256);
        mbar_init(B_OFULL, 1);
        fence_mbar_init();
        tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
    }
    if (warp == 9) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int n_items = a.n_qtiles * a.KVH * a.splits;
    const int kv_valid = prefill_kv_valid(a);

    // Key-tile range of a query tile (identical in every role); tiles count KEYS logical positions.
    auto tile_span = [&](int qt, int sp, int& kt_lo, int& nt) { prefill_tile_span(a, a.QT, KEYS, qt, sp, kt_lo, nt); };

    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        // K and V travel through separate rings: a K tile is free again as soon as its score MMA
        // has run (long before P·V of the same tile), and V has one more stage than K where shared
        // memory allows, so the loads of tile t+2 never wait for the output MMA of tile t.
        if (lane == 0) {
            uint32_t gt = 0, it = 0, q_it = 0;
            bool ok = true, q_pending = false;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
                const int sp = item % a.splits, rest = item / a.splits;
                const int qt = a.n_qtiles - 1 - rest / a.KVH, kvh = rest % a.KVH;  // longest spans first
                int kt_lo, nt;
                tile_span(qt, sp, kt_lo, nt);
                if (!mbar_wait(B_QEMPTY, (it & 1) ^ 1, a.status)) { ok = false; break; }
                mbar_expect_tx(B_QFULL, (uint32_t)(NCH * a.QT * a.G * 128));
#pragma unroll
                for (int c = 0; c < NCH; ++c)
                    tma_load_3d(q_smem + c * Q_CHUNK, &tm_q, B_QFULL, c * 64, kvh * a.G, qt * a.QT);
                q_pending = true;
                q_it = it;
                for (int t = 0; t < nt; ++t, ++gt) {
                    const int row = prefill_tile_row(a, (kt_lo + t) * KEYS);
                    const uint32_t ks = gt % KST, ku = gt / KST;
                    if (!mbar_wait(B_KEMPTY + 8 * ks, (ku & 1) ^ 1, a.status)) { ok = false; break; }
                    mbar_expect_tx(B_KFULL + 8 * ks, KV_TILE);
#pragma unroll
                    for (int c = 0; c < NCH; ++c)
                        tma_load_4d(k_smem + ks * KV_TILE + c * KV_CHUNK, &tm_k, B_KFULL + 8 * ks, c * 64, kvh, row, 0);
                    const uint32_t vs = gt % VST, vu = gt / VST;
                    if (!mbar_wait(B_VEMPTY + 8 * vs, (vu & 1) ^ 1, a.status)) {
                        // the K copy above is in flight: wait for it before giving up
                        mbar_wait(B_KFULL + 8 * ks, ku & 1, a.status);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(B_VFULL + 8 * vs, KV_TILE);
#pragma unroll
                    for (int c = 0; c < NCH; ++c)
                        tma_load_4d(v_smem + vs * KV_TILE + c * KV_CHUNK, &tm_v, B_VFULL + 8 * vs, c * 64, kvh, row, 0);
                }
            }
            // drain this thread's outstanding copies before the CTA retires (tiles 0..gt-1 were issued)
            if (q_pending) mbar_wait(B_QFULL, q_it & 1, a.status);
            for (uint32_t i = 1; i <= (uint32_t)KST && i <= gt; ++i) {
                const uint32_t g = gt - i;
                mbar_wait(B_KFULL + 8 * (g % KST), (g / KST) & 1, a.status);
            }
            for (uint32_t i = 1; i <= (uint32_t)VST && i <= gt; ++i) {
                const uint32_t g = gt - i;
                mbar_wait(B_VFULL + 8 * (g % VST), (g / VST) & 1, a.status);
            }
        }
    } else if (warp == 9) {
        // ------------------------------ MMA issuer ------------------------------
        // Issue order per item: QK(0), QK(1), PV(0), QK(2), PV(1), ... — the score MMA of tile t+1
        // runs while the softmax warps work on tile t.
        if (lane == 0) {
            uint32_t gt = 0, it = 0;
            bool ok = true;
            const int ksteps = (a.HD + 15) / 16;   // k-steps holding real dimensions (the zero-filled ones are skipped)
            auto issue_qk = [&](uint32_t g) -> bool {
                const uint32_t ks = g % KST, sb = g & 1;
                if (!mbar_wait(B_KFULL + 8 * ks, (g / KST) & 1, a.status) ||
                    !mbar_wait(B_SFREE + 8 * sb, ((g >> 1) & 1) ^ 1, a.status))
                    return false;
                tc_fence_after();
                const uint32_t kbase = k_smem + ks * KV_TILE;
                const uint32_t d = tmem + (sb ? COL_S1 : COL_S0);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    if (kk < ksteps)
                        tc_mma_ss(d, umma_desc_sw128(q_smem + (kk / 4) * Q_CHUNK + (kk % 4) * 32, 16),
                                  umma_desc_sw128(kbase + (kk / 4) * KV_CHUNK + (kk % 4) * 32, 16), IDESC_QK, kk > 0);
                }
                tc_commit(B_SFULL + 8 * sb);
                tc_commit(B_KEMPTY + 8 * ks);   // the K tile is free once these MMAs have run
                return true;
            };
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
                const int sp = item % a.splits, rest = item / a.splits;
                const int qt = a.n_qtiles - 1 - rest / a.KVH;
                int kt_lo, nt;
                tile_span(qt, sp, kt_lo, nt);
                if (!mbar_wait(B_QFULL, it & 1, a.status) || !issue_qk(gt)) { ok = false; break; }
                for (int t = 0; t < nt && ok; ++t, ++gt) {
                    if (t + 1 < nt) {
                        if (!issue_qk(gt + 1)) { ok = false; break; }
                    } else {
                        tc_commit(B_QEMPTY);  // last score MMA of the item issued: Q tile may be replaced
                    }
                    const uint32_t vs = gt % VST;
                    if (!mbar_wait(B_PFULL, gt & 1, a.status) ||
                        !mbar_wait(B_VFULL + 8 * vs, (gt / VST) & 1, a.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    // O accumulates in tensor memory over the whole item (the first tile overwrites)
                    const uint32_t vbase = v_smem + vs * KV_TILE;
                    const uint32_t pbase = tmem + ((gt & 1) ? COL_P1 : COL_P0);
#pragma unroll
                    for (int kk = 0; kk < KEYS / 16; ++kk)
                        tc_mma_ts(tmem + COL_PV, pbase + kk * 8, umma_desc_sw128(vbase + kk * 2048, KV_CHUNK),
                                  IDESC_PV, (t > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(B_PVFULL);
                    if (t + 1 == nt) tc_commit(B_OFULL);   // the item's output is complete
                    tc_commit(B_VEMPTY + 8 * vs);
                }
            }
            // every MMA issued above has completed before tensor memory is freed
            tc_commit(B_DONE);
            mbar_wait(B_DONE, 0, a.status);
        }
    } else {
        // ------------------------------ softmax / output rows ------------------------------
        // Two threads per row: warps 0-3 take the first half of the score tile's columns and of the
        // output dimensions, warps 4-7 the other halves. Tensor-memory lanes are reached through
        // the warp's quadrant (warp % 4).
        const int quad = warp & 3, half = warp >> 2;
        const int r = quad * 32 + lane;            // row of the tile = lane of tensor memory
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        constexpr int HH = HD / 2;                 // output dimensions per thread
        const int ql = r / a.G, g = r % a.G;
        uint32_t gt = 0, xn = 0, si = 0;   // tiles seen, exchanges done, items done (barrier phases)
        bool ok = true;            // kept warp-uniform: a wait that ran out for any lane stops the warp
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int sp = item % a.splits, rest = item / a.splits;
            const int qt = a.n_qtiles - 1 - rest / a.KVH, kvh = rest % a.KVH;
            int kt_lo, nt;
            tile_span(qt, sp, kt_lo, nt);
            const int qi = qt * a.QT + ql;
            const bool row_valid = ql < a.QT && qi < a.S_new;
            const int qpos = a.past_len + qi;
            const int first_row = a.window > 0 ? (qpos + 1 - a.window > 0 ? qpos + 1 - a.window : 0) : 0;
            const int qlim = prefill_last_key(a, qpos);  // never attend rows past a linear plane
            // m_ref: the reference maximum the probabilities and O are scaled by. It only moves
            // when a tile's maximum exceeds it by more than 2^8 (then O is rescaled in tensor
            // memory); otherwise P simply carries the factor, which fp16 holds comfortably.
            float m_ref = kNegBig, l_run = 0.0f;

            for (int t = 0; t < nt; ++t, ++gt) {
                const uint32_t sb = gt & 1;
                const uint32_t s_addr = tmem + lane_sel + (sb ? COL_S1 : COL_S0) + half * KH;
                const int kstart = (kt_lo + t) * KEYS + half * KH;   // key of this thread's column 0
                ok = __all_sync(0xffffffffu, ok && mbar_wait(B_SFULL + 8 * sb, (gt >> 1) & 1, a.status));
                if (!ok) continue;
                tc_fence_after();
                uint32_t sv[KH];
#pragma unroll
                for (int c = 0; c < KH / 32; ++c) tmem_ld32(*reinterpret_cast<uint32_t (*)[32]>(&sv[c * 32]), s_addr + c * 32);
                tc_wait_ld();
                // columns [lo, hi] of this thread's KH are attended (causal + window)
                const int lo = first_row - kstart, hi = qlim - kstart;
                const bool all_in = __all_sync(0xffffffffu, lo <= 0 && hi >= KH - 1);
                // the maximum is taken on the raw scores (the scale is positive) and scaled once
                float mx = -INFINITY;
                if (all_in) {
#pragma unroll
                    for (int j = 0; j < KH; j += 2)
                        mx = fmax3(mx, __uint_as_float(sv[j]), __uint_as_float(sv[j + 1]));
                } else {
#pragma unroll
                    for (int j = 0; j < KH; ++j) {
                        const float s = (j >= lo && j <= hi) ? __uint_as_float(sv[j]) : -INFINITY;
                        sv[j] = __float_as_uint(s);
                        mx = fmaxf(mx, s);
                    }
                }
                mx *= a.scale_log2;
                // row maximum over both halves
                xch[(sb * 2 + half) * kPfRows + r] = mx;
                mbar_arrive(B_XCH);
                ok = __all_sync(0xffffffffu, mbar_wait(B_XCH, xn & 1, a.status));
                ++xn;
                if (!ok) continue;
                mx = fmaxf(mx, xch[(sb * 2 + (half ^ 1)) * kPfRows + r]);
                const bool move = mx > m_ref + 8.0f;
                if (__any_sync(0xffffffffu, move)) {
                    const float m_to = move ? mx : m_ref;
                    const float alpha = exp2f(m_ref - m_to);   // 1 for rows that keep their reference
                    if (t > 0) {
                        // rescale this thread's half of O in place; every earlier P·V must have landed.
                        // (The parity wait is sound here: the score MMA of this tile was issued after
                        // P·V of tile t-2, so the barrier is at most one phase behind.)
                        ok = __all_sync(0xffffffffu, mbar_wait(B_PVFULL, (gt - 1) & 1, a.status));
                        if (!ok) continue;
                        tc_fence_after();
                        tmem_scale_columns(tmem + lane_sel + COL_PV + half * HH, HH / 32, alpha);
                    }
                    l_run *= alpha;
                    m_ref = m_to;
                }
                // p = 2^(s*scale - m_ref): one packed FMA, two ex2, one packed add, one pack per pair
                float lsum0 = 0.0f, lsum1 = 0.0f;
                const float neg_m = -m_ref;
                uint32_t pk[KH / 2];
#pragma unroll
                for (int j = 0; j < KH; j += 2) {
                    float x0, x1;
                    ffma2_bcast(x0, x1, __uint_as_float(sv[j]), __uint_as_float(sv[j + 1]), a.scale_log2, neg_m);
                    const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                    fadd2_acc(lsum0, lsum1, p0, p1);
                    pk[j / 2] = pack_half2(p0, p1);
                }
                const float lsum = lsum0 + lsum1;
                {
                    const uint32_t pcol = (sb ? COL_P1 : COL_P0) + half * (KH / 2);
#pragma unroll
                    for (int c = 0; c < KH / 32; ++c)
                        tmem_st16(tmem + lane_sel + pcol + c * 16, *reinterpret_cast<uint32_t (*)[16]>(&pk[c * 16]));
                }
                tc_wait_st();
                l_run += lsum;
                // cache rows of this tile past the last written position may hold stale bits:
                // zero them in the staged V tile so that 0 * garbage cannot produce NaN
                const int tile0 = (kt_lo + t) * KEYS;
                if (tile0 + KEYS > kv_valid) {
                    const uint32_t vs = gt % VST;
                    ok = __all_sync(0xffffffffu, mbar_wait(B_VFULL + 8 * vs, (gt / VST) & 1, a.status));
                    if (!ok) continue;
                    uint8_t* vt = v_gen + (size_t)vs * KV_TILE;
                    const int first_bad = kv_valid > tile0 ? kv_valid - tile0 : 0;
                    for (int idx = first_bad * 8 * NCH + tid; idx < KEYS * 8 * NCH; idx += 256) {
                        const int row = idx / (8 * NCH), u = idx % (8 * NCH);
                        *reinterpret_cast<uint4*>(vt + (u / 8) * KV_CHUNK + row * 128 + (u % 8) * 16) =
                            make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                tc_fence_before();
                mbar_arrive(B_SFREE + 8 * sb);
                mbar_arrive(B_PFULL);
            }
            // total row sum = both halves' partial sums (same reference maximum)
            float l_tot = l_run;
            if (ok) {
                xch[4 * kPfRows + half * kPfRows + r] = l_run;
                mbar_arrive(B_XCH);
                ok = __all_sync(0xffffffffu, mbar_wait(B_XCH, xn & 1, a.status));
                ++xn;
                l_tot += xch[4 * kPfRows + (half ^ 1) * kPfRows + r];
            }
            // Wait for the item's last P·V, then write this thread's half of the row out, 32 columns
            // at a time. This is a barrier of its own with one phase per item: the per-tile barrier
            // may still be two phases behind here (nothing orders P·V of tile nt-2 before this
            // point), where a parity wait passes a phase early.
            ok = __all_sync(0xffffffffu, ok && mbar_wait(B_OFULL, si & 1, a.status));
            ++si;
            if (!ok) continue;
            tc_fence_after();
            const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
            float* prow = nullptr;
            __half* op = nullptr;
            if (row_valid) {
                const int parts = a.out_parts > 0 ? a.out_parts : a.splits;
                const int part = a.out_parts > 0 ? a.out_part * a.splits + sp : sp;
                if (parts > 1) prow = a.part + (((long long)qi * a.part_stride + part) * a.H + (long long)kvh * a.G + g) * (a.HD + 2);
                else op = a.out + ((long long)qi * a.H + (long long)kvh * a.G + g) * a.HD;
            }
#pragma unroll
            for (int c = 0; c < HH / 32; ++c) {
                const int d0 = half * HH + c * 32;     // first output dimension of this piece
                uint32_t v[32];
                tmem_ld32(v, tmem + lane_sel + COL_PV + d0);
                tc_wait_ld();
                if (d0 >= a.HD) continue;              // zero-filled padding columns (head_dim 96)
                if (prow) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2)
                        *reinterpret_cast<float2*>(prow + d0 + j) = make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                } else if (op) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 w;
                        w.x = pack_half2(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
                        w.y = pack_half2(__uint_as_float(v[j + 2]) * inv, __uint_as_float(v[j + 3]) * inv);
                        w.z = pack_half2(__uint_as_float(v[j + 4]) * inv, __uint_as_float(v[j + 5]) * inv);
                        w.w = pack_half2(__uint_as_float(v[j + 6]) * inv, __uint_as_float(v[j + 7]) * inv);
                        *reinterpret_cast<uint4*>(op + d0 + j) = w;
                    }
                }
            }
            if (prow && half == 0) {
                prow[a.HD] = m_ref;
                prow[a.HD + 1] = l_tot;
            }
            tc_fence_before();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Merge of the key-range partials written by the kernel above: one warp per (query, head) row,
// each lane HD/32 output dimensions. The partial rows are [o(HD), m (log2 domain), l] in fp32.
// ---------------------------------------------------------------------------
// With `row_parts` the count of partials is read per (query, kv head) — rows with a single part were
// written in final form by the attention kernel and are left alone.
__global__ void __launch_bounds__(256) hkv_prefill_combine_kernel(const float* __restrict__ part,
                                                                  __half* __restrict__ out, long long rows,
                                                                  int H, int HD, int splits, int part_stride,
                                                                  const int* __restrict__ row_parts, int G) {
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const long long qi = row / H;
    const int head = (int)(row % H);
    if (row_parts) {
        splits = row_parts[qi * (H / G) + head / G];
        if (splits <= 1) return;
    }
    const long long stride = (long long)H * (HD + 2);
    const float* base = part + (qi * part_stride * H + head) * (HD + 2);
    float M = kNegBig;
    for (int sp = 0; sp < splits; ++sp) M = fmaxf(M, __ldg(base + sp * stride + HD));
    // lane l takes the dimension pairs 2l, 2l + 64, ... (head_dim is even; rows are 8-byte aligned)
    float L = 0.0f, acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    for (int sp = 0; sp < splits; ++sp) {
        const float* r = base + sp * stride;
        const float w = exp2f(__ldg(r + HD) - M);
        L = fmaf(__ldg(r + HD + 1), w, L);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int d = lane * 2 + 64 * j;
            if (d < HD) {
                const float2 v = __ldg(reinterpret_cast<const float2*>(r + d));
                acc[2 * j] = fmaf(v.x, w, acc[2 * j]);
                acc[2 * j + 1] = fmaf(v.y, w, acc[2 * j + 1]);
            }
        }
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int d = lane * 2 + 64 * j;
        if (d < HD) *reinterpret_cast<uint32_t*>(out + row * HD + d) = pack_half2(acc[2 * j] * inv, acc[2 * j + 1] * inv);
    }
}

}  // namespace hkv
