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
// (sequence, token, head), no block-wide barrier.
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

constexpr int kRopeWarps = 4;

// Unit of work u = ((b*S + s) * (H + 2*KVH) + j): j < H query head, j < H+KVH key head,
// else value head (copy only, when a cache is given).
__global__ void __launch_bounds__(kRopeWarps * 32) hkv_qk_norm_rope_kernel(const RopeArgs a) {
    __shared__ float s_x[kRopeWarps][512];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tok = a.H + 2 * a.KVH;
    const long long units = (long long)a.B * a.S * per_tok;
    for (long long u = (long long)blockIdx.x * kRopeWarps + warp; u < units;
         u += (long long)gridDim.x * kRopeWarps) {
        const int j = (int)(u % per_tok);
        const long long tok = u / per_tok;
        const int s = (int)(tok % a.S), b = (int)(tok / a.S);
        const int pos = (a.d_pos ? a.d_pos[b * a.pos_stride] : a.host_pos) + s;
        const bool is_q = j < a.H, is_k = !is_q && j < a.H + a.KVH;
        const int kvh = is_q ? 0 : (is_k ? j - a.H : j - a.H - a.KVH);
        int slot = -1;
        if (!is_q && a.k_cache) {
            slot = slot_of_pos(a.map, pos);
            if (slot < 0) continue;  // dropped past the plane / owned by another rank
        }
        const long long cache_off =
            (long long)b * a.batch_stride + ((long long)slot * a.KVH + kvh) * a.HD;
        if (!is_q && !is_k) {  // value head: plain copy into the cache
            if (!a.k_cache || !a.v) continue;
            const __half* src = a.v + ((tok * a.KVH) + kvh) * a.HD;
            for (int i = lane; i < a.HD; i += 32) a.v_cache[cache_off + i] = src[i];
            continue;
        }
        const __half* src = is_q ? a.q + (tok * a.H + j) * a.HD : a.k + (tok * a.KVH + kvh) * a.HD;
        __half* dst = is_q ? a.q + (tok * a.H + j) * a.HD
                           : (a.k_cache ? a.k_cache + cache_off : a.k + (tok * a.KVH + kvh) * a.HD);
        const __half* w = is_q ? a.q_w : a.k_w;
        float* x = s_x[warp];
        float ssq = 0.0f;
        for (int i = lane; i < a.HD; i += 32) {
            const float t = __half2float(src[i]);
            x[i] = t;
            ssq = fmaf(t, t, ssq);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        const float inv = 1.0f / sqrtf(ssq / (float)a.HD + a.eps);
        __syncwarp();
        for (int i = lane; i < a.HD; i += 32) x[i] = x[i] * inv * __half2float(w[i]);
        __syncwarp();
        const int half_rot = a.rot / 2;
        const float fp = (float)pos / a.scaling;
        for (int i = lane; i < a.HD; i += 32) {
            if (i < half_rot) {
                const float freq = 1.0f / powf(a.theta, (float)(2 * i) / (float)a.rot);
                float sn, c;
                sincosf(fp * freq, &sn, &c);
                const float x0 = x[i], x1 = x[i + half_rot];
                dst[i] = __float2half_rn(x0 * c - x1 * sn);
                dst[i + half_rot] = __float2half_rn(x0 * sn + x1 * c);
            } else if (i >= a.rot) {
                dst[i] = __float2half_rn(x[i]);
            }
        }
        __syncwarp();
    }
}

}  // namespace hkv
