// hkv_basic.cuh — append, any-geometry split-K decode, combine and synthetic fill.
//
// Reference semantics restated here (paths relative to the reference project root):
//   append   kernels/attention.cu:1119-1151   decode  kernels/attention.cu:337-494
#pragma once

#include "hkv_common.cuh"

namespace hkv {

// ---------------------------------------------------------------------------
// Append: K and V rows of `seq_new` tokens per sequence in ONE launch.
// One thread per VEC-byte piece of a (sequence, token, plane) row of KVH*HD halfs.
// VEC = 16 when every pointer/stride allows it, else 2.
// ---------------------------------------------------------------------------
struct AppendArgs {
    const __half* k_new;
    const __half* v_new;
    __half* k_cache;
    __half* v_cache;
    const int32_t* d_pos;  // [B] or null -> host_pos
    int pos_stride;        // 1: d_pos[b]; 0: every sequence reads d_pos[0] (the reference's scalar)
    int host_pos;
    int pos_bias;          // added to the position read from d_pos (e.g. -1: length -> index)
    SeqMap map;
    int B, S, row_elems;   // row_elems = KVH*HD
    long long batch_stride;
    long long src_stride;  // elements between sequences in k_new / v_new (S*row_elems when dense)
};

template <typename VecT>
__global__ void __launch_bounds__(256) hkv_append_kernel(const AppendArgs a) {
    constexpr int kPer = (int)(sizeof(VecT) / sizeof(__half));
    const int pieces = a.row_elems / kPer;  // per row
    const long long total = 2ll * a.B * a.S * pieces;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int piece = (int)(i % pieces);
        long long r = i / pieces;
        const int plane = (int)(r & 1);
        r >>= 1;
        const int s = (int)(r % a.S);
        const int b = (int)(r / a.S);
        const int pos = (a.d_pos ? a.d_pos[b * a.pos_stride] + a.pos_bias : a.host_pos) + s;
        const int slot = slot_of_pos(a.map, pos);
        if (slot < 0) continue;
        const __half* src = (plane ? a.v_new : a.k_new) + (long long)b * a.src_stride + (long long)s * a.row_elems;
        __half* dst = (plane ? a.v_cache : a.k_cache) + (long long)b * a.batch_stride +
                      (long long)slot * a.row_elems;
        reinterpret_cast<VecT*>(dst)[piece] = reinterpret_cast<const VecT*>(src)[piece];
    }
}

// ---------------------------------------------------------------------------
// Generic split-K decode (SIMT). One CTA of 4 warps per (chunk, head, sequence);
// warp w takes rows lo+w, lo+w+4, ... of the chunk; lane-strided dot product and
// online softmax per warp in the log2 domain; warps merged in shared memory; one
// partial (m, l, o[HD]) per (sequence, chunk, head). Any head_dim <= 512, any group.
// ---------------------------------------------------------------------------
constexpr int kGenWarps = 4;
constexpr int kGenMaxPerLane = 16;  // head_dim <= 512

__global__ void __launch_bounds__(kGenWarps * 32) hkv_decode_generic_kernel(const DecodeArgs a) {
    const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = attended_len(a, b);
    int tile_lo, n_tiles;
    tile_range(a.map, total, tile_lo, n_tiles);
    const int n_chunks = (n_tiles + a.chunk_tiles - 1) / a.chunk_tiles;
    if (chunk >= n_chunks) return;

    const int G = a.H / a.KVH;
    const int kvh = h / G;
    const int first = first_pos(a.map, total);
    const int row0 = (tile_lo + chunk * a.chunk_tiles) * kTileRows;
    int row1 = row0 + a.chunk_tiles * kTileRows;
    const int row_end = (tile_lo + n_tiles) * kTileRows;
    if (row1 > row_end) row1 = row_end;
    if (row1 > a.map.slots) row1 = a.map.slots;

    float qr[kGenMaxPerLane], acc[kGenMaxPerLane];
    const __half* qp = a.q + (long long)b * a.q_stride + (long long)h * a.HD;
#pragma unroll
    for (int i = 0; i < kGenMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        qr[i] = d < a.HD ? __half2float(qp[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = kNegBig, l = 0.0f;
    const long long plane_off = (long long)b * a.batch_stride + (long long)kvh * a.HD;
    const int row_elems = a.KVH * a.HD;

    for (int s = row0 + warp; s < row1; s += kGenWarps) {
        const int p = pos_of_slot(a.map, s, total);
        if (p < first || p >= total) continue;  // warp-uniform
        const __half* kr = a.k_cache + plane_off + (long long)s * row_elems;
        const __half* vr = a.v_cache + plane_off + (long long)s * row_elems;
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < kGenMaxPerLane; ++i) {
            const int d = lane + 32 * i;
            if (d < a.HD) dot = fmaf(qr[i], __half2float(kr[d]), dot);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float sc = dot * a.scale_log2;
        const float mn = fmaxf(m, sc);
        const float corr = exp2f(m - mn), e = exp2f(sc - mn);
        l = l * corr + e;
#pragma unroll
        for (int i = 0; i < kGenMaxPerLane; ++i) {
            const int d = lane + 32 * i;
            if (d < a.HD) acc[i] = fmaf(e, __half2float(vr[d]), acc[i] * corr);
        }
        m = mn;
    }

    __shared__ float s_m[kGenWarps], s_l[kGenWarps];
    __shared__ float s_acc[kGenWarps][kGenMaxPerLane * 32];
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < kGenMaxPerLane; ++i) s_acc[warp][lane + 32 * i] = acc[i];
    __syncthreads();

    float gm = s_m[0];
#pragma unroll
    for (int w = 1; w < kGenWarps; ++w) gm = fmaxf(gm, s_m[w]);
    float gl = 0.0f;
#pragma unroll
    for (int w = 0; w < kGenWarps; ++w) gl += s_l[w] * exp2f(s_m[w] - gm);
    float* prow = a.part + (((long long)b * a.max_chunks + chunk) * a.H + h) * (a.HD + 2);
    for (int d = threadIdx.x; d < a.HD; d += kGenWarps * 32) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kGenWarps; ++w) o += s_acc[w][d] * exp2f(s_m[w] - gm);
        prow[d] = o;
    }
    if (threadIdx.x == 0) {
        prow[a.HD] = gm;
        prow[a.HD + 1] = gl;
    }
}

// ---------------------------------------------------------------------------
// Combine: merge the partials of one (sequence, head).
//   o = sum_c 2^(m_c - M) o_c,  l = sum_c 2^(m_c - M) l_c,  M = max_c m_c
// A partial is a row of HD+2 floats (o[0..HD), m, l); partial c of (b, h) starts at
// part[b*stride_b + c*stride_c + h*(HD+2)]. Count: from the sequence length (local
// split-K) or fixed (partials gathered from other GPUs).
// Output: fp16 rows (RN, zero when l == 0 — kernels/attention.cu:478) and/or one merged
// partial [B, H, HD+2] for the cross-GPU exchange.
// ---------------------------------------------------------------------------
struct CombineArgs {
    const float* part;
    long long stride_b, stride_c;  // floats
    const int32_t* total;          // null -> host_len (or fixed_count when that is > 0)
    int pos_is_index;
    int pos_stride;                // as DecodeArgs
    int host_len;
    int fixed_count;               // > 0: that many partials per row, whatever the length
    // Equal-span schedule (span_spans > 0): sequence b's partials sit at slots span + b for the spans
    // that overlap its tiles, found from the tile table the decode kernel left in gpre.
    const int* gpre;               // [B+1]
    int span_spans;                // spans the decode launch was given (grid / gang)
    int B;
    SeqMap map;
    int chunk_tiles;
    int H, HD;
    __half* out;         // [B, H, HD] or null
    float* out_partial;  // [B, H, HD+2] or null
    // Peer exchange (pub_n > 0): the merged partial goes to this rank's own mailbox (local memory, the
    // parity of the current epoch), where the peers READ it once the merge kernel of this rank has
    // released the epoch.
    int pub_n = 0;
    float* pub_part = nullptr;       // parity 0 of the partial area of this rank's mailbox
    long long pub_parity_stride = 0; // floats between the two parities
    const uint32_t* pub_state = nullptr;   // this rank's epoch counter (advanced by the merge kernel)
};

// Epoch of the exchange a publishing launch belongs to.
__device__ __forceinline__ uint32_t pub_epoch(const CombineArgs& a) {
    return a.pub_n ? *reinterpret_cast<const volatile uint32_t*>(a.pub_state) : 0u;
}
__device__ __forceinline__ void store_partial(const CombineArgs& a, const uint32_t epoch, const long long idx, const float v) {
    if (a.out_partial) a.out_partial[idx] = v;
    if (a.pub_n) a.pub_part[(long long)(epoch & 1u) * a.pub_parity_stride + idx] = v;
}

constexpr int kCombineWarps = 8;
constexpr int kCombineThreads = kCombineWarps * 32;

// One CTA per (head, sequence). The partials are dealt to the warps (warp w takes c = w, w+8, ...);
// a warp reads one partial row at a time, lane l the output dimensions l, l+32, ... — coalesced
// 128-byte pieces, several rows in flight — so the merge is bandwidth- rather than latency-bound
// even when a single sequence has 128 partials and only `heads` CTAs exist. Warps then reduce
// through shared memory.
__global__ void __launch_bounds__(kCombineThreads) hkv_combine_kernel(const CombineArgs a) {
    const int h = blockIdx.x, b = blockIdx.y;
    const int PW = a.HD + 2;
    int n;
    const float* base;
    long long stride_c = a.stride_c;
    if (a.span_spans > 0) {
        const int p0 = a.gpre[b], p1 = a.gpre[b + 1], W = a.gpre[a.B];
        const int spans = span_count(W, a.span_spans);
        const int first = p1 > p0 ? span_owner(p0, W, spans) : 0;
        n = p1 > p0 ? span_owner(p1 - 1, W, spans) - first + 1 : 0;
        stride_c = (long long)a.H * PW;
        base = a.part + ((long long)(first + b) * a.H + h) * PW;
    } else {
        n = a.fixed_count > 0
                ? a.fixed_count
                : num_chunks(a.map, length_of(a.total, a.pos_stride, a.pos_is_index, a.host_len, b), a.chunk_tiles);
        base = a.part + b * a.stride_b + (long long)h * PW;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t epoch = pub_epoch(a);
    __shared__ float s_max[kCombineWarps];
    __shared__ float s_sum[kCombineWarps];
    __shared__ float s_acc[kCombineWarps][512];   // head_dim <= 512
    // One pass: a warp folds its rows into a running (maximum, sum, row) — no separate pass for the
    // maximum, so the launch is one round trip shorter — four rows' loads in flight at a time.
    const int ndim = (a.HD + 31) >> 5;   // dimensions per lane, <= 16
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
    float Mw = kNegBig, Lw = 0.0f;
    for (int c0 = warp; c0 < n; c0 += 4 * kCombineWarps) {
        float m[4], l[4], x[4][16];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = c0 + u * kCombineWarps;
            const float* row = base + (long long)(c < n ? c : c0) * stride_c;
            m[u] = c < n ? row[a.HD] : kNegBig;
            l[u] = c < n ? row[a.HD + 1] : 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int d = lane + 32 * i;
                x[u][i] = (i < ndim && d < a.HD && c < n) ? row[d] : 0.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float Mn = fmaxf(Mw, m[u]);
            const float keep = exp2f(Mw - Mn), w = exp2f(m[u] - Mn);
            Lw = fmaf(l[u], w, Lw * keep);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (i < ndim) acc[i] = fmaf(x[u][i], w, acc[i] * keep);
            Mw = Mn;
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int d = lane + 32 * i;
        if (i < ndim && d < a.HD) s_acc[warp][d] = acc[i];
    }
    if (lane == 0) {
        s_max[warp] = Mw;
        s_sum[warp] = Lw;
    }
    __syncthreads();
    float M = s_max[0];
#pragma unroll
    for (int w = 1; w < kCombineWarps; ++w) M = fmaxf(M, s_max[w]);
    float wgt[kCombineWarps];
    float L = 0.0f;
#pragma unroll
    for (int w = 0; w < kCombineWarps; ++w) {
        wgt[w] = exp2f(s_max[w] - M);
        L = fmaf(s_sum[w], wgt[w], L);
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    for (int d = tid; d < a.HD; d += kCombineThreads) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kCombineWarps; ++w) o = fmaf(s_acc[w][d], wgt[w], o);
        if (a.out) a.out[((long long)b * a.H + h) * a.HD + d] = __float2half_rn(o * inv);
        store_partial(a, epoch, ((long long)b * a.H + h) * PW + d, o);
    }
    if (tid == 0) {
        store_partial(a, epoch, ((long long)b * a.H + h) * PW + a.HD, M);
        store_partial(a, epoch, ((long long)b * a.H + h) * PW + a.HD + 1, L);
    }
}

// The merge for many (sequence, head) rows: one thread per output dimension walks the row's
// partials directly; no cross-warp reduction and half the threads of the kernel above, which only
// pays when few rows each have many partials (small batches).
__global__ void __launch_bounds__(128) hkv_combine_few_kernel(const CombineArgs a) {
    const int h = blockIdx.x, b = blockIdx.y;
    const int PW = a.HD + 2;
    int n;
    const float* base;
    long long stride_c = a.stride_c;
    if (a.span_spans > 0) {
        const int p0 = a.gpre[b], p1 = a.gpre[b + 1], W = a.gpre[a.B];
        const int spans = span_count(W, a.span_spans);
        const int first = p1 > p0 ? span_owner(p0, W, spans) : 0;
        n = p1 > p0 ? span_owner(p1 - 1, W, spans) - first + 1 : 0;
        stride_c = (long long)a.H * PW;
        base = a.part + ((long long)(first + b) * a.H + h) * PW;
    } else {
        n = a.fixed_count > 0
                ? a.fixed_count
                : num_chunks(a.map, length_of(a.total, a.pos_stride, a.pos_is_index, a.host_len, b), a.chunk_tiles);
        base = a.part + b * a.stride_b + (long long)h * PW;
    }
    const int tid = threadIdx.x;
    const uint32_t epoch = pub_epoch(a);
    // Every thread reads the row's n (maximum, sum) pairs itself — the same addresses across the CTA, so
    // they are broadcast from L1 — and needs no exchange with the others: no shared memory, no barrier.
    float M = kNegBig;
#pragma unroll 4
    for (int c = 0; c < n; ++c) M = fmaxf(M, base[(long long)c * stride_c + a.HD]);
    float L = 0.0f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // output dims tid, tid+128, ... (head_dim <= 512)
#pragma unroll 4
    for (int c = 0; c < n; ++c) {
        const float* row = base + (long long)c * stride_c;
        const float w = exp2f(row[a.HD] - M);
        L = fmaf(row[a.HD + 1], w, L);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = tid + 128 * i;
            if (d < a.HD) acc[i] = fmaf(row[d], w, acc[i]);
        }
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int d = tid + 128 * i;
        if (d < a.HD) {
            if (a.out) a.out[((long long)b * a.H + h) * a.HD + d] = __float2half_rn(acc[i] * inv);
            store_partial(a, epoch, ((long long)b * a.H + h) * PW + d, acc[i]);
        }
    }
    if (threadIdx.x == 0) {
        store_partial(a, epoch, ((long long)b * a.H + h) * PW + a.HD, M);
        store_partial(a, epoch, ((long long)b * a.H + h) * PW + a.HD + 1, L);
    }
}

// ---------------------------------------------------------------------------
// Merge of published partials: both halves of the peer exchange's handshake.
//   1. The first CTA to arrive releases this rank's partial of the current epoch: one system-scope
//      fence, then the new epoch stored into the flag word this rank owns in every rank's mailbox
//      (4-byte stores over NVLink). The partial was written by the launch before this one on the
//      stream, so it is complete; nothing of the publishing kernels pays for fences or counters.
//   2. Every CTA waits — with a bound — until the flag of every rank in THIS rank's mailbox has reached
//      the epoch, then one warp per (sequence, head) row reads that epoch's partial of every rank — its
//      own from local memory, the others' through their peer-mapped mailboxes over NVLink (plain
//      system-scope loads, nothing cached) — and merges them.
//   3. The last CTA to finish advances the epoch counter for the next exchange.
// When the wait runs out the rows are left untouched, the status word gets kStatusWaitRanOut and the
// kernel returns normally (the epoch still advances); launches that find the bit already set do not wait.
// ---------------------------------------------------------------------------
struct MergePublishedArgs {
    const float* part[kMaxPeers];   // parity 0 of rank r's partial area, as mapped here: [2][rows][HD+2]
    uint32_t* flag_out[kMaxPeers];  // this rank's flag word in rank r's mailbox
    const uint32_t* flags;          // [world] in this rank's mailbox, written by the peers
    uint32_t* state;                // this rank's {epoch, CTAs finished, CTAs arrived}
    int world, rows, HD;
    __half* out;                    // [rows][HD]
    int32_t* status;
    unsigned long long limit_ns;
};

constexpr int kMergeWarps = 4;

__device__ __forceinline__ float ld_sys(const float* p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kMergeWarps * 32) hkv_merge_published_kernel(const MergePublishedArgs a) {
    __shared__ int s_ok;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t expect = *reinterpret_cast<const volatile uint32_t*>(a.state) + 1u;
    if (tid == 0) {
        if (atomicAdd(a.state + 2, 1u) == 0u) {          // first to arrive: release this rank's partial
            __threadfence_system();
            for (int r = 0; r < a.world; ++r)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flag_out[r]), "r"(expect) : "memory");
        }
        // a wait that already ran out (an earlier layer of this step) is not repeated: a lost peer costs
        // one limit per step, not one per layer
        s_ok = (*reinterpret_cast<volatile int32_t*>(a.status) & kStatusWaitRanOut) ? 0 : 1;
    }
    __syncthreads();
    if (s_ok && tid < a.world) {
        unsigned long long t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (;;) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.flags + tid) : "memory");
            if ((int32_t)(seen - expect) >= 0) break;
            __nanosleep(100);
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > a.limit_ns) {
                atomicOr(a.status, kStatusWaitRanOut);
                s_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    const int row = blockIdx.x * kMergeWarps + warp;
    if (s_ok && row < a.rows) {
        const int PW = a.HD + 2;
        const long long at = (long long)((expect - 1u) & 1u) * a.rows * PW + (long long)row * PW;
        // the two scalars of every rank first (lanes 0..world-1 fetch them in parallel), then the rows
        float m_r = kNegBig, l_r = 0.0f;
        if (lane < a.world) {
            m_r = ld_sys(a.part[lane] + at + a.HD);
            l_r = ld_sys(a.part[lane] + at + a.HD + 1);
        }
        float M = m_r;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        const float w_r = lane < a.world ? exp2f(m_r - M) : 0.0f;
        float L = l_r * w_r;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        // The rows, 128 dimensions at a time: the loads of ALL ranks are issued before the first is used, so the
        // merge pays about one NVLink round trip per slab instead of one per rank.
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
        float wr[kMaxPeers];
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) wr[r] = __shfl_sync(0xffffffffu, w_r, r);
#pragma unroll
        for (int slab = 0; slab < 4; ++slab) {
            if (slab * 128 >= a.HD) break;
            float v[kMaxPeers][4];
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int d = slab * 128 + lane + 32 * i;
                    v[r][i] = (r < a.world && d < a.HD) ? ld_sys(a.part[r] + at + d) : 0.0f;
                }
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[slab * 4 + i] = fmaf(v[r][i], wr[r], acc[slab * 4 + i]);
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int d = lane + 32 * i;
            if (d < a.HD) a.out[(long long)row * a.HD + d] = __float2half_rn(acc[i] * inv);
        }
    }
    // the last CTA to finish closes the exchange: the next publishing launch reads the new epoch
    __syncthreads();
    if (tid == 0 && atomicAdd(a.state + 1, 1u) == gridDim.x - 1) {
        a.state[1] = 0;
        a.state[2] = 0;
        *reinterpret_cast<volatile uint32_t*>(a.state) = expect;
    }
}

// ---------------------------------------------------------------------------
// Self-test of the bounded wait: one CTA waits on an mbarrier that nothing ever arrives on.
// The wait must run out after `limit_ns`, set the status word and let the kernel return
// normally, so the host can see how a lost producer would surface. No trap, no endless loop.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(32) hkv_selftest_wait_kernel(int32_t* status, unsigned long long limit_ns,
                                                               int32_t* waited_ok) {
    __shared__ uint64_t bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        fence_mbar_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait(b, 0, status, limit_ns);  // phase 0 never completes
        if (waited_ok) *waited_ok = ok ? 1 : 0;
    }
}

// ---------------------------------------------------------------------------
// Synthetic data (same bits as the CPU generator of the test oracle): the sum of
// twelve 16-bit uniform fields of three splitmix64 outputs, centred and scaled by an
// exact power of two (Irwin-Hall(12): mean 0, variance 1), rounded RN to fp16.
// ---------------------------------------------------------------------------
__host__ __device__ inline unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__global__ void __launch_bounds__(256) hkv_fill_kernel(__half* dst, unsigned long long seed,
                                                       unsigned long long first,
                                                       unsigned long long count) {
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x;
         i < count; i += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned long long base = splitmix64(seed ^ ((first + i) * 0xD1342543DE82EF95ull));
        unsigned int sum = 0;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const unsigned long long v = splitmix64(base + (unsigned long long)r);
            sum += (unsigned int)(v & 0xFFFF) + (unsigned int)((v >> 16) & 0xFFFF) +
                   (unsigned int)((v >> 32) & 0xFFFF) + (unsigned int)((v >> 48) & 0xFFFF);
        }
        const float x = (float)((int)(2u * sum) - 786420) * (1.0f / 131072.0f);
        dst[i] = __float2half_rn(x);
    }
}

}  // namespace hkv
