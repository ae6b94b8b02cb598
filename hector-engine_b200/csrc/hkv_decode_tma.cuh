// hkv_decode_tma.cuh — split-K flash-decode for B200: K/V tiles staged into shared
// memory by bulk-tensor (TMA) loads behind an mbarrier pipeline, every KV head shared by
// its whole query group inside one CTA, online softmax with warp-shuffle reductions.
//
// Replaces attention_cached_v2_kernel_dp (reference kernels/attention.cu:337-494), which
// runs one 512-thread CTA per (sequence, query head), re-reads each KV head once per
// query head of its group and issues 4-byte loads.
//
// Shape of the computation
//   * Persistent grid (one or two CTAs per SM) under an equal-span schedule: the 64-row tiles of all
//     sequences of the batch form one line (the lengths are read on the device), cut into as many
//     equal contiguous spans as there are gangs of CTAs. A gang is `span_gang` neighbouring CTAs that
//     share a span, each taking its own KV heads — so the gang streams neighbouring bytes in step and
//     every CTA of the launch does the same number of tile steps whatever the batch and the lengths
//     are: no quantisation over the SMs, no tail, and a sequence is cut only where a span ends (one
//     partial per (span, sequence) instead of one per fixed-size chunk).
//   * Warp NCW (last) is the producer: one lane walks the CTA's item list and issues,
//     per tile, HD/CW box loads for K and for V ([64 rows] x [CW halfs], 128- or 64-byte
//     swizzle) into a ring of `stages` buffers. It runs ahead across item boundaries,
//     so the memory pipe never drains between items.
//   * Consumer warps work in groups of four; tile i of the CTA's stream belongs to
//     group i % NGROUPS, warp w of the group owns rows [16w, 16w+16) of the tile.
//     Scores:  S^T[16 rows x 8 heads] = K_tile · Q^T   (mma m16n8k16, A = K via
//     ldmatrix, B = Q held in registers; the query group sits in the N dimension, so a
//     group of 7 wastes 1/8 of the tile, not 9/16).
//     Softmax over rows: per-head max via shuffles (xor 4, 8, 16), log2 domain.
//     Output:  O^T[HD x 8 heads] += V_tile^T · P^T    (A = V^T via ldmatrix.trans,
//     B = P^T obtained from the score fragment with movmatrix).
//   * At the end of a piece (the part of a sequence inside the span) the consumer warps merge
//     their (m, l, O) in shared memory and write one partial row per head at slot span + sequence
//     (distinct for every piece, as both only grow along the line); the combine kernel finds a
//     sequence's partials from the same arithmetic and finishes the softmax.
//   * Fused append: the warp that owns the row of the new token patches the staged tile
//     from k_new/v_new and stores the row into the cache plane; rows that are staged but
//     not attended (tail of the last tile, outside the window) are masked, and their V
//     rows zeroed in shared memory so stale bits can never reach the accumulators.
//   * Every barrier wait is bounded; on expiry the status word is set and the CTA drains
//     its own outstanding copies and returns.
#pragma once

#include <cuda.h>

#include "hkv_common.cuh"

namespace hkv {

constexpr int kMaxStages = 8;
constexpr int kTmaMaxBatch = 4096;  // prefix table lives in shared memory

struct TmaSmemPlan {
    int stages;
    size_t bytes;  // dynamic shared memory to request (includes alignment slack)
};

__host__ __device__ constexpr int tma_chunk_width(int HD) { return HD % 64 == 0 ? 64 : 32; }

// Shared-memory plan: as many stages as fit under `budget` bytes.
inline TmaSmemPlan tma_plan(int HD, int G, int ncw, int B, size_t budget) {
    const size_t stage = 2ull * kTileRows * HD * 2;
    const size_t fixed = 1024 /*align*/ + (size_t)ncw * G * (HD + 4) * 4 + (size_t)ncw * G * 2 * 4 +
                         2 * kMaxStages * 8 + (size_t)(B + 1) * 4 + 64;
    int s = (int)((budget > fixed ? budget - fixed : 0) / stage);
    if (s > kMaxStages) s = kMaxStages;
    // Tile i of a CTA's stream uses stage i % stages and belongs to consumer group
    // i % groups. The stage count must be a multiple of the group count so that a stage
    // (and its full barrier) always serves the same group: otherwise a group could run a
    // whole barrier phase ahead of the other and a parity wait would pass on stale data.
    const int groups = ncw / 4;
    s -= s % groups;
    return TmaSmemPlan{s, fixed + (size_t)s * stage};
}

// NGROUPS = 2: one CTA per SM, two consumer groups sharing one deep ring (long launches).
// NGROUPS = 1: TWO CTAs per SM, each with one consumer group and a ring of half the depth: while one
// CTA merges an item or waits for its first tiles, the other keeps the SM's memory pipe busy — the
// fixed cost per launch (ramp and tail) that dominates short launches is overlapped instead of paid
// twice. The host picks by the amount of work per SM.
// STALE: the plane is a ring larger than its window (see tma_tile_range); its bookkeeping is compiled
// into the kernels that need it only, the others keep their registers.
template <int HD, int NT, int NGROUPS, bool STALE = false>
__global__ void __launch_bounds__((NGROUPS * 4 + 1) * 32, NGROUPS == 1 ? 2 : 1)
hkv_decode_tma_kernel(const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const DecodeArgs a,
                      const int stages) {
    constexpr int CW = tma_chunk_width(HD);
    constexpr int NCH = HD / CW;
    constexpr int ROWB = CW * 2;
    constexpr int CHUNK_BYTES = kTileRows * ROWB;
    constexpr int TILE_BYTES = kTileRows * HD * 2;
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    constexpr int NCW = NGROUPS * 4;
    constexpr int KS = HD / 16;  // k-steps of QK^T == m-tiles of PV
    constexpr int OS = HD + 4;   // merge row stride (floats): conflict-free fragment stores

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int G = a.H / a.KVH;
    float* mrg_o = reinterpret_cast<float*>(smem + (size_t)stages * STAGE_BYTES);  // [NCW][G][OS]
    float* mrg_ml = mrg_o + (size_t)NCW * G * OS;                                  // [NCW][G][2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(mrg_ml + (size_t)NCW * G * 2);
    int* prefix = reinterpret_cast<int*>(bars + 2 * kMaxStages);                   // [B+1]
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kMaxStages);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 4);
        }
        fence_mbar_init();
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    // prefix[b] = tiles of the sequences before b. Warp 0 scans the batch 32 sequences at a time
    // with shuffles (a serial scan by one thread costs a microsecond at batch 64, in front of the
    // first load of every launch).
    if (warp == 0) {
        int carry = 0;
        for (int b0 = 0; b0 < a.B; b0 += 32) {
            const int b = b0 + lane;
            int v = 0, tl, wt;
            if (b < a.B) {
                if (STALE) tma_tile_range(a.map, attended_len(a, b), tl, v, wt);
                else tile_range(a.map, attended_len(a, b), tl, v);
            }
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += u;
            }
            if (b < a.B) prefix[b + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        if (lane == 0) prefix[0] = 0;
    }
    __syncthreads();
    // This CTA's span of the line and its share of the KV heads.
    const int W = prefix[a.B];
    if (blockIdx.x == 0)   // the combine kernel finds each sequence's partials from the same table
        for (int b = tid; b <= a.B; b += blockDim.x) a.gpre[b] = prefix[b];
    const int GS = a.span_gang;
    const int NS = span_count(W, (int)gridDim.x / GS);
    const int span = blockIdx.x / GS, member = blockIdx.x % GS;
    int u0 = 0, u1 = 0, b_first = 0;
    if (span < NS) {
        u0 = (int)((long long)W * span / NS);
        u1 = (int)((long long)W * (span + 1) / NS);
        int lo = 0, hi = a.B - 1;          // the sequence that holds tile u0
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (prefix[mid] <= u0) lo = mid; else hi = mid - 1;
        }
        b_first = lo;
    }

    if (warp == NCW) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            int stage = 0, round = 0, issued = 0;
            bool ok = true;
            for (int kvh = member; kvh < a.KVH && ok; kvh += GS) {
                int b = b_first;
                for (int u = u0; u < u1 && ok; ++b) {
                    const int nb = prefix[b + 1] - prefix[b];
                    if (nb == 0) continue;             // an empty sequence (free batch slot)
                    const int off = u - prefix[b];
                    const int nt = nb - off < u1 - u ? nb - off : u1 - u;
                    int tile_lo, n_tiles, wrap_tiles = 0x7fffffff;
                    if (STALE) tma_tile_range(a.map, attended_len(a, b), tile_lo, n_tiles, wrap_tiles);
                    else tile_range(a.map, attended_len(a, b), tile_lo, n_tiles);
                    const int t0 = tile_lo + off;
                    u += nt;
                    for (int t = 0; t < nt; ++t) {
                        if (round > 0 &&
                            !mbar_wait(empty0 + 8 * stage, (uint32_t)(round - 1) & 1u, a.status)) {
                            ok = false;
                            break;
                        }
                        const uint32_t full = full0 + 8 * stage;
                        const uint32_t dst = smem_base + (uint32_t)stage * STAGE_BYTES;
                        mbar_expect_tx(full, STAGE_BYTES);
                        const int row = ((STALE && t0 + t >= wrap_tiles) ? t0 + t - wrap_tiles : t0 + t) * kTileRows;
#pragma unroll
                        for (int c = 0; c < NCH; ++c)
                            tma_load_4d(dst + c * CHUNK_BYTES, &tm_k, full, c * CW, kvh, row, b);
#pragma unroll
                        for (int c = 0; c < NCH; ++c)
                            tma_load_4d(dst + TILE_BYTES + c * CHUNK_BYTES, &tm_v, full, c * CW, kvh,
                                        row, b);
                        ++issued;
                        if (++stage == stages) { stage = 0; ++round; }
                    }
                }
            }
            // Drain: every copy this thread issued has landed before the CTA retires.
            // (In a clean run the consumers already waited on them; this returns at once.)
            const int back = issued < stages ? issued : stages;
            for (int i = 0; i < back; ++i) {
                if (--stage < 0) { stage = stages - 1; --round; }
                mbar_wait(full0 + 8 * stage, (uint32_t)round & 1u, a.status);
            }
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
    const int grp = warp >> 2, wig = warp & 3;
    const int r4 = lane >> 2, c4 = lane & 3;
    // ldmatrix lane geometry (row inside the tile, 16-byte unit select)
    const int k_row = wig * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;   // K: matrices 1,3 are rows+8
    const int k_sel = lane >> 4;                                       // K: matrices 2,3 are k+8
    const int v_row = wig * 16 + (lane & 7) + (lane >> 4) * 8;         // V^T: matrices 2,3 are rows+8
    const int v_sel = (lane >> 3) & 1;                                 // V^T: matrices 1,3 are d+8
    const int k_swz = (CW == 64) ? (k_row & 7) : ((k_row >> 1) & 3);
    const int v_swz = (CW == 64) ? (v_row & 7) : ((v_row >> 1) & 3);

    int stage = 0, round = 0, tile_seq = 0;
    bool ok = true;
    for (int kvh = member; kvh < a.KVH; kvh += GS)
    for (int b = b_first, u = u0; u < u1; ++b) {
        const int nb = prefix[b + 1] - prefix[b];
        if (nb == 0) continue;                 // an empty sequence (free batch slot)
        const int off = u - prefix[b];
        const int nt = nb - off < u1 - u ? nb - off : u1 - u;
        u += nt;
        const int total = attended_len(a, b);
        int tile_lo, n_tiles, row_lo, row_hi, wrap_tiles = 0x7fffffff;
        if (STALE) tma_tile_range(a.map, total, tile_lo, n_tiles, wrap_tiles);
        else tile_range(a.map, total, tile_lo, n_tiles);
        slot_range(a.map, total, row_lo, row_hi);
        const int first = first_pos(a.map, total);
        const int t0 = tile_lo + off;
        // A ring that has wrapped holds an attended position in EVERY row when the window spans the whole
        // ring (what a sliding-window layer allocates): no row of any tile needs checking. A ring larger than
        // its window keeps stale rows outside the window: its tiles are checked, cheaply — positions along a
        // wrapped ring follow from the row of the newest position (the seam) without a division per row.
        const bool ring_wrapped = STALE && a.map.layout == 1 && total > a.map.slots;
        const bool ring_stale_rows = ring_wrapped && a.map.window > 0 && a.map.window < a.map.slots;
        // (without STALE a wrapped ring larger than its window still decodes correctly: every tile checked row by row)
        const bool always_mask = (!STALE && a.map.layout == 1 && total > a.map.slots && a.map.window > 0 && a.map.window < a.map.slots) ||
                                 (a.map.shard_count > 1 && a.map.window > 0);
        int seam = 0, ring_base = 0;
        if (ring_wrapped) {
            seam = (total - 1) % a.map.slots;
            ring_base = total - 1 - seam;
        }
        auto pos_at = [&](int s) {
            return ring_wrapped ? ring_base + s - (s > seam ? a.map.slots : 0) : pos_of_slot(a.map, s, total);
        };
        const int new_slot = a.k_new ? slot_of_pos(a.map, total - 1) : -1;

        // Query fragments: B operand [16 d x 8 heads], head = r4, d pair = c4*2 (+8).
        uint32_t qb[NT][KS][2];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int head = n * 8 + r4;
            const __half* qp = a.q + (long long)b * a.q_stride + ((long long)kvh * G + head) * HD;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                if (head < G) {
                    qb[n][ks][0] = *reinterpret_cast<const uint32_t*>(qp + ks * 16 + c4 * 2);
                    qb[n][ks][1] = *reinterpret_cast<const uint32_t*>(qp + ks * 16 + c4 * 2 + 8);
                } else {
                    qb[n][ks][0] = 0u;
                    qb[n][ks][1] = 0u;
                }
            }
        }
        float m_run[NT][2], l_run[NT][2], o_acc[NT][KS][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            m_run[n][0] = m_run[n][1] = kNegBig;
            l_run[n][0] = l_run[n][1] = 0.0f;
#pragma unroll
            for (int mt = 0; mt < KS; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) o_acc[n][mt][e] = 0.0f;
        }

        for (int t = 0; t < nt; ++t) {
            const bool mine = (tile_seq % NGROUPS) == grp;
            ++tile_seq;
            // After a wait has run out this warp stops waiting and computing but keeps
            // walking the item list, so that it still meets the others at the merge barrier.
            if (mine && ok && !mbar_wait(full0 + 8 * stage, (uint32_t)round & 1u, a.status))
                ok = false;
            if (mine && ok) {
                const uint32_t kbase = smem_base + (uint32_t)stage * STAGE_BYTES;
                const uint32_t vbase = kbase + TILE_BYTES;
                uint8_t* kgen = smem + (size_t)stage * STAGE_BYTES;
                uint8_t* vgen = kgen + TILE_BYTES;
                const int row0 = ((STALE && t0 + t >= wrap_tiles) ? t0 + t - wrap_tiles : t0 + t) * kTileRows;
                bool masked = always_mask || row0 < row_lo || row0 + kTileRows > row_hi;
                if (ring_stale_rows)   // whole tile inside the window: rows run upward from row0's position, no seam inside
                    masked = (seam >= row0 && seam < row0 + kTileRows - 1) || row0 + kTileRows > a.map.slots || pos_at(row0) < first;
                bool touched = false;

                if (masked) {
                    // zero the V rows of this warp that are staged but not attended
                    for (int r = 0; r < 16; ++r) {
                        const int s = row0 + wig * 16 + r;
                        const int p = pos_at(s);
                        const bool valid = s < a.map.slots && p >= first && p < total;
                        if (!valid) {
                            const int tr = wig * 16 + r;
                            const int swz = (CW == 64) ? (tr & 7) : ((tr >> 1) & 3);
                            for (int u = lane; u < HD / 8; u += 32) {
                                const int c = (u * 8) / CW, uu = (u * 8 % CW) / 8;
                                *reinterpret_cast<uint4*>(vgen + c * CHUNK_BYTES + tr * ROWB +
                                                          ((uu ^ swz) << 4)) = make_uint4(0, 0, 0, 0);
                            }
                            touched = true;
                        }
                    }
                }
                if (new_slot >= row0 + wig * 16 && new_slot < row0 + wig * 16 + 16) {
                    // fused append: stage the new row and store it into the cache planes
                    const int tr = new_slot - row0;
                    const int swz = (CW == 64) ? (tr & 7) : ((tr >> 1) & 3);
                    const long long src = (long long)b * a.new_stride + (long long)kvh * HD;
                    const long long dst = (long long)b * a.batch_stride +
                                          ((long long)new_slot * a.KVH + kvh) * HD;
                    for (int u = lane; u < HD / 8; u += 32) {
                        const int c = (u * 8) / CW, uu = (u * 8 % CW) / 8;
                        const uint32_t off = c * CHUNK_BYTES + tr * ROWB + ((uu ^ swz) << 4);
                        const uint4 kv = *reinterpret_cast<const uint4*>(a.k_new + src + u * 8);
                        const uint4 vv = *reinterpret_cast<const uint4*>(a.v_new + src + u * 8);
                        *reinterpret_cast<uint4*>(kgen + off) = kv;
                        *reinterpret_cast<uint4*>(vgen + off) = vv;
                        *reinterpret_cast<uint4*>(a.k_cache_w + dst + u * 8) = kv;
                        *reinterpret_cast<uint4*>(a.v_cache_w + dst + u * 8) = vv;
                    }
                    touched = true;
                }
                if (touched) __syncwarp();

                // ---- scores: S^T = K · Q^T --------------------------------------
                float sc[NT][2][4];
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) sc[n][0][e] = sc[n][1][e] = 0.0f;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const int d0 = ks * 16 + k_sel * 8;
                    const int c = d0 / CW, u = (d0 % CW) / 8;
                    uint32_t a0, a1, a2, a3;
                    ldsm_x4(kbase + c * CHUNK_BYTES + k_row * ROWB + ((u ^ k_swz) << 4), a0, a1, a2, a3);
#pragma unroll
                    for (int n = 0; n < NT; ++n)
                        mma_16816(sc[n][ks & 1], a0, a1, a2, a3, qb[n][ks][0], qb[n][ks][1]);
                }

                // ---- online softmax over rows, per head column -------------------
                bool vA = true, vB = true;
                if (masked) {
                    const int sA = row0 + wig * 16 + r4, sB = sA + 8;
                    const int pA = pos_at(sA), pB = pos_at(sB);
                    vA = sA < a.map.slots && pA >= first && pA < total;
                    vB = sB < a.map.slots && pB >= first && pB < total;
                }
                uint32_t pb[NT][2];
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    float s0 = (sc[n][0][0] + sc[n][1][0]) * a.scale_log2;
                    float s1 = (sc[n][0][1] + sc[n][1][1]) * a.scale_log2;
                    float s2 = (sc[n][0][2] + sc[n][1][2]) * a.scale_log2;
                    float s3 = (sc[n][0][3] + sc[n][1][3]) * a.scale_log2;
                    if (!vA) { s0 = -INFINITY; s1 = -INFINITY; }
                    if (!vB) { s2 = -INFINITY; s3 = -INFINITY; }
                    float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
                    for (int o = 4; o <= 16; o <<= 1) {
                        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
                    }
                    const float mn0 = fmaxf(m_run[n][0], mx0), mn1 = fmaxf(m_run[n][1], mx1);
                    const float al0 = exp2f(m_run[n][0] - mn0), al1 = exp2f(m_run[n][1] - mn1);
                    const float p0 = exp2f(s0 - mn0), p1 = exp2f(s1 - mn1);
                    const float p2 = exp2f(s2 - mn0), p3 = exp2f(s3 - mn1);
                    m_run[n][0] = mn0;
                    m_run[n][1] = mn1;
                    l_run[n][0] = l_run[n][0] * al0 + p0 + p2;
                    l_run[n][1] = l_run[n][1] * al1 + p1 + p3;
#pragma unroll
                    for (int mt = 0; mt < KS; ++mt) {
                        o_acc[n][mt][0] *= al0;
                        o_acc[n][mt][1] *= al1;
                        o_acc[n][mt][2] *= al0;
                        o_acc[n][mt][3] *= al1;
                    }
                    // P^T as B operand: transpose the two 8x8 score blocks in registers
                    pb[n][0] = movmatrix_t(pack_half2(p0, p1));
                    pb[n][1] = movmatrix_t(pack_half2(p2, p3));
                }

                // ---- output: O^T += V^T · P^T -------------------------------------
#pragma unroll
                for (int mt = 0; mt < KS; ++mt) {
                    const int d0 = mt * 16 + v_sel * 8;
                    const int c = d0 / CW, u = (d0 % CW) / 8;
                    uint32_t a0, a1, a2, a3;
                    ldsm_x4_t(vbase + c * CHUNK_BYTES + v_row * ROWB + ((u ^ v_swz) << 4), a0, a1, a2, a3);
#pragma unroll
                    for (int n = 0; n < NT; ++n)
                        mma_16816(o_acc[n][mt], a0, a1, a2, a3, pb[n][0], pb[n][1]);
                }

                if (touched) fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * stage);
            }
            if (++stage == stages) { stage = 0; ++round; }
        }
        // ---- merge the consumer warps, write one partial row per head -----------
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
                l_run[n][0] += __shfl_xor_sync(0xffffffffu, l_run[n][0], o);
                l_run[n][1] += __shfl_xor_sync(0xffffffffu, l_run[n][1], o);
            }
            const int h0 = n * 8 + c4 * 2;
#pragma unroll
            for (int mt = 0; mt < KS; ++mt) {
                const int d = mt * 16 + r4;
                if (h0 < G) {
                    mrg_o[((size_t)warp * G + h0) * OS + d] = o_acc[n][mt][0];
                    mrg_o[((size_t)warp * G + h0) * OS + d + 8] = o_acc[n][mt][2];
                }
                if (h0 + 1 < G) {
                    mrg_o[((size_t)warp * G + h0 + 1) * OS + d] = o_acc[n][mt][1];
                    mrg_o[((size_t)warp * G + h0 + 1) * OS + d + 8] = o_acc[n][mt][3];
                }
            }
            if (r4 == 0) {
                if (h0 < G) {
                    mrg_ml[((size_t)warp * G + h0) * 2] = m_run[n][0];
                    mrg_ml[((size_t)warp * G + h0) * 2 + 1] = l_run[n][0];
                }
                if (h0 + 1 < G) {
                    mrg_ml[((size_t)warp * G + h0 + 1) * 2] = m_run[n][1];
                    mrg_ml[((size_t)warp * G + h0 + 1) * 2 + 1] = l_run[n][1];
                }
            }
        }
        named_bar_sync(1, NCW * 32);
        float* prow = a.span_part + ((long long)(span + b) * a.H + (long long)kvh * G) * (HD + 2);
        for (int idx = tid; idx < G * HD; idx += NCW * 32) {
            const int g = idx / HD, d = idx % HD;
            float M = kNegBig;
#pragma unroll
            for (int w = 0; w < NCW; ++w) M = fmaxf(M, mrg_ml[((size_t)w * G + g) * 2]);
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < NCW; ++w)
                o = fmaf(mrg_o[((size_t)w * G + g) * OS + d],
                         exp2f(mrg_ml[((size_t)w * G + g) * 2] - M), o);
            prow[(long long)g * (HD + 2) + d] = o;
        }
        if (tid < G) {
            float M = kNegBig, L = 0.0f;
#pragma unroll
            for (int w = 0; w < NCW; ++w) M = fmaxf(M, mrg_ml[((size_t)w * G + tid) * 2]);
#pragma unroll
            for (int w = 0; w < NCW; ++w)
                L += mrg_ml[((size_t)w * G + tid) * 2 + 1] * exp2f(mrg_ml[((size_t)w * G + tid) * 2] - M);
            prow[(long long)tid * (HD + 2) + HD] = M;
            prow[(long long)tid * (HD + 2) + HD + 1] = L;
        }
        named_bar_sync(1, NCW * 32);
    }
}

}  // namespace hkv
