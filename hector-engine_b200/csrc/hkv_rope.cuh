// hkv_rope.cuh — per-head RMSNorm of q and k + rotary embedding, with the rotated K and the
// V row written straight into the cache planes (the front of the append path).
//
// Replaces qk_norm_rope_kernel<DEVICE_POS, WRITE_CACHE> and its launchers (reference
// kernels/attention.cu:800-973): same arithmetic
//   x_n[i] = x[i] * rsqrt(mean(x^2) + eps) * w[i]
//   pairs (i, i + rot/2), i < rot/2, rotated by ((s + pos) / scaling) / theta^(2i/rot)
//   dims >= rot pass through normalised
// but batched over sequences with one device position per sequence, row lookup through
// the same position->row map as the append (linear drop / ring / shard owner), one warp per
// (sequence, token, head), the rotation table computed once per token and CTA, 8-byte accesses.
#pragma once

#include "hkv_common.cuh"

namespace hkv {

struct RopeArgs {
    __half* q;              // [B, S, H, HD], rewritten in place
    __half* k;              // [B, S, KVH, HD]: rewritten in place when k_cache is null
    const __half* v;        // [B, S, KVH, HD] or null
    const __half* q_w;      // [HD]
    const __half* k_w;      // [HD]
    __half* k_cache;        // [B, slots, KVH, HD] or null
    __half* v_cache;
    const int32_t* d_pos;   // [B] or null -> host_pos
    int pos_stride;         // 1: d_pos[b]; 0: every sequence reads d_pos[0]
    int host_pos;
    SeqMap map;
    int B, S, H, KVH, HD, rot;
    long long batch_stride;
    float eps, theta, scaling;
};

constexpr int kRopeWarps = 8;

// One unit of one token (see the kernel below); `x` is the calling warp's fp32 staging row.
__device__ __forceinline__ void rope_unit(const RopeArgs& a, const int vec, const long long tok, const int b, const int pos,
                                          const int j, const int per_tok, const int half_rot, float* x,
                                          const float (*s_w)[512], const float* s_cos, const float* s_sin, const int lane) {
    if (j >= per_tok) return;
    const bool is_q = j < a.H, is_k = !is_q && j < a.H + a.KVH;
    const int kvh = is_q ? 0 : (is_k ? j - a.H : j - a.H - a.KVH);
    int slot = -1;
    if (!is_q && a.k_cache) {
        slot = slot_of_pos(a.map, pos);
        if (slot < 0) return;  // dropped past the plane / owned by another rank
    }
    const long long cache_off = (long long)b * a.batch_stride + ((long long)slot * a.KVH + kvh) * a.HD;
    if (!is_q && !is_k) {  // value head: plain copy into the cache
        if (!a.k_cache || !a.v) return;
        const __half* src = a.v + ((tok * a.KVH) + kvh) * a.HD;
        __half* dst = a.v_cache + cache_off;
        if (vec) {
            for (int i = lane; i < a.HD / 4; i += 32) reinterpret_cast<uint2*>(dst)[i] = reinterpret_cast<const uint2*>(src)[i];
        } else {
            for (int i = lane; i < a.HD; i += 32) dst[i] = src[i];
        }
        return;
    }
    const __half* src = is_q ? a.q + (tok * a.H + j) * a.HD : a.k + (tok * a.KVH + kvh) * a.HD;
    __half* dst = is_q ? a.q + (tok * a.H + j) * a.HD
                       : (a.k_cache ? a.k_cache + cache_off : a.k + (tok * a.KVH + kvh) * a.HD);
    const float* w = s_w[is_q ? 0 : 1];
    float ssq = 0.0f;
    if (vec) {
        for (int i = lane; i < a.HD / 4; i += 32) {
            const uint2 raw = reinterpret_cast<const uint2*>(src)[i];
            const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            x[4 * i] = lo.x; x[4 * i + 1] = lo.y; x[4 * i + 2] = hi.x; x[4 * i + 3] = hi.y;
            ssq = fmaf(lo.x, lo.x, fmaf(lo.y, lo.y, fmaf(hi.x, hi.x, fmaf(hi.y, hi.y, ssq))));
        }
    } else {
        for (int i = lane; i < a.HD; i += 32) {
            const float t = __half2float(src[i]);
            x[i] = t;
            ssq = fmaf(t, t, ssq);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    const float inv = 1.0f / sqrtf(ssq / (float)a.HD + a.eps);
    __syncwarp();
    // normalised value of element e, and its rotated image
    auto norm = [&](int e) { return x[e] * inv * w[e]; };
    auto rotated = [&](int e) {
        if (e < half_rot) return norm(e) * s_cos[e] - norm(e + half_rot) * s_sin[e];
        if (e < a.rot) return norm(e - half_rot) * s_sin[e - half_rot] + norm(e) * s_cos[e - half_rot];
        return norm(e);
    };
    if (vec) {
        for (int i = lane; i < a.HD / 4; i += 32) {
            uint2 o;
            o.x = pack_half2(rotated(4 * i), rotated(4 * i + 1));
            o.y = pack_half2(rotated(4 * i + 2), rotated(4 * i + 3));
            reinterpret_cast<uint2*>(dst)[i] = o;
        }
    } else {
        for (int i = lane; i < a.HD; i += 32) dst[i] = __float2half_rn(rotated(i));
    }
}

// A work item is kRopeWarps units of ONE token: a unit is a query head, a key head or a value head
// (j < H query head j, j < H + KVH key head, else value head — a plain copy, only when a cache is
// given). Items are numbered token-major; every CTA takes a contiguous range of them, so it loads
// the norm weights once and recomputes the rotation table only when its token changes.
//   * The rotation angles depend on (position, pair index) only, so a CTA computes the cos/sin
//     table of a token once (rot/2 entries, accurate powf + sincosf: positions reach 10^5 rad)
//     and every head of the token reuses it — the reference recomputes it per head and per pair.
//   * Rows move in 8-byte pieces (4 halfs per lane: a 128-wide head is one piece per lane) when the
//     pointers and head_dim allow it, else element by element. A warp stages its head as fp32 in
//     shared memory, so any rotary_dim <= head_dim <= 512 takes the same code.
__global__ void __launch_bounds__(kRopeWarps * 32) hkv_qk_norm_rope_kernel(const RopeArgs a, const int vec) {
    __shared__ float s_x[kRopeWarps][512];
    __shared__ float s_cos[256], s_sin[256];
    __shared__ float s_w[2][512];          // q and k norm weights as fp32
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tok = a.H + 2 * a.KVH;
    const int groups = (per_tok + kRopeWarps - 1) / kRopeWarps;       // items per token
    const long long items = (long long)a.B * a.S * groups;
    const long long i0 = items * blockIdx.x / gridDim.x, i1 = items * (blockIdx.x + 1) / gridDim.x;
    const int half_rot = a.rot / 2;
    for (int i = threadIdx.x; i < a.HD; i += blockDim.x) {
        s_w[0][i] = __half2float(a.q_w[i]);
        s_w[1][i] = __half2float(a.k_w[i]);
    }
    long long table_tok = -1;
    for (long long item = i0; item < i1; ++item) {
    const long long tok = item / groups;
    const int s = (int)(tok % a.S), b = (int)(tok / a.S);
    const int pos = (a.d_pos ? a.d_pos[b * a.pos_stride] : a.host_pos) + s;
    if (tok != table_tok) {                 // block-uniform
        __syncthreads();                    // the previous token's table is no longer being read
        const float fp = (float)pos / a.scaling;
        for (int i = threadIdx.x; i < half_rot; i += blockDim.x) {
            const float freq = 1.0f / powf(a.theta, (float)(2 * i) / (float)a.rot);
            float sn, c;
            sincosf(fp * freq, &sn, &c);
            s_cos[i] = c;
            s_sin[i] = sn;
        }
        __syncthreads();
        table_tok = tok;
    }
    rope_unit(a, vec, tok, b, pos, (int)(item % groups) * kRopeWarps + warp, per_tok, half_rot, s_x[warp], s_w, s_cos, s_sin, lane);
    }
}

}  // namespace hkv
