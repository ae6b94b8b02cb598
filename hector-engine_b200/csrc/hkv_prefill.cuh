// hkv_prefill.cuh — attention of a chunk of new queries over the cache (batch 1).
//
// Semantics of the reference's attention_prefill_cached_kernel
// (kernels/attention.cu:664-773): query i attends cache rows [first_i, past_len + i] with
// first_i = window > 0 ? max(0, past_len + i + 1 - window) : 0; the cache already holds
// the chunk's own K/V rows.
#pragma once

#include "hkv_basic.cuh"

namespace hkv {

struct PrefillArgs {
    const __half* q;        // [S_new, H, HD]
    const __half* k_cache;  // [slots, KVH, HD]
    const __half* v_cache;
    __half* out;            // [S_new, H, HD]
    int S_new, past_len, H, KVH, HD, slots, window;
    int ring;               // 1: position p lives in row p % slots
    float scale_log2;
};

// Any-geometry SIMT kernel: one CTA of 4 warps per (query, head), rows dealt to warps
// round-robin, online softmax per warp, merge in shared memory, fp16 RN output.
__global__ void __launch_bounds__(kGenWarps * 32) hkv_prefill_generic_kernel(const PrefillArgs a) {
    const int qi = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = a.H / a.KVH, kvh = h / G;
    int total = a.past_len + qi + 1;
    const int first = a.window > 0 ? (total - a.window > 0 ? total - a.window : 0) : 0;
    if (!a.ring && total > a.slots) total = a.slots;   // a linear plane drops rows past its end

    float qr[kGenMaxPerLane], acc[kGenMaxPerLane];
    const __half* qp = a.q + ((long long)qi * a.H + h) * a.HD;
#pragma unroll
    for (int i = 0; i < kGenMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        qr[i] = d < a.HD ? __half2float(qp[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = kNegBig, l = 0.0f;
    const int row_elems = a.KVH * a.HD;
    for (int s = first + warp; s < total; s += kGenWarps) {
        const int row = a.ring ? s % a.slots : s;
        const __half* kr = a.k_cache + (long long)row * row_elems + kvh * a.HD;
        const __half* vr = a.v_cache + (long long)row * row_elems + kvh * a.HD;
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
    const float inv = gl > 0.0f ? 1.0f / gl : 0.0f;
    __half* op = a.out + ((long long)qi * a.H + h) * a.HD;
    for (int d = threadIdx.x; d < a.HD; d += kGenWarps * 32) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kGenWarps; ++w) o += s_acc[w][d] * exp2f(s_m[w] - gm);
        op[d] = __float2half_rn(o * inv);
    }
}

}  // namespace hkv
