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

// One unit of one token through shared memory, element by element: any alignment, any rotary_dim
// (see the kernel below); `x` is the calling warp's fp32 staging row.
__device__ __forceinline__ void rope_unit_scalar(const RopeArgs& a, const __half* src, __half* dst, const float* w,
                                                 const int half_rot, float* x, const float* s_cos, const float* s_sin,
                                                 const int lane) {
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
    auto norm = [&](int e) { return x[e] * inv * w[e]; };
    for (int i = lane; i < a.HD; i += 32) {
        float r;
        if (i < half_rot) r = norm(i) * s_cos[i] - norm(i + half_rot) * s_sin[i];
        else if (i < a.rot) r = norm(i - half_rot) * s_sin[i - half_rot] + norm(i) * s_cos[i - half_rot];
        else r = norm(i);
        dst[i] = __float2half_rn(r);
    }
    __syncwarp();
}

// One unit of one token in registers: lane l holds the 4-element pieces l, l + 32, ... of the head
// (8-byte loads and stores); the rotation partner of a piece sits rot/8 pieces away — in another lane
// (one shuffle per value) or, for wide heads, in the same lane's other piece. Needs head_dim and
// rotary_dim/2 to be multiples of 4 and at most 32 pieces between partners' lanes... see `fast` below.
template <int PIECES>   // pieces per lane: head_dim <= 128 * PIECES
__device__ __forceinline__ void rope_unit_vec(const RopeArgs& a, const __half* src, __half* dst, const float* w,
                                              const int half_rot, const float* s_cos, const float* s_sin, const int lane) {
    const int P = a.HD / 4, hp = half_rot / 4, rp = a.rot / 4;   // pieces per row, per half rotation, in the rotated part
    float x[PIECES][4];
    float ssq = 0.0f;
#pragma unroll
    for (int k = 0; k < PIECES; ++k) {
        const int i = lane + 32 * k;
        if (i < P) {
            const uint2 raw = reinterpret_cast<const uint2*>(src)[i];
            const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            x[k][0] = lo.x; x[k][1] = lo.y; x[k][2] = hi.x; x[k][3] = hi.y;
            ssq = fmaf(lo.x, lo.x, fmaf(lo.y, lo.y, fmaf(hi.x, hi.x, fmaf(hi.y, hi.y, ssq))));
        } else {
            x[k][0] = x[k][1] = x[k][2] = x[k][3] = 0.0f;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    const float inv = 1.0f / sqrtf(ssq / (float)a.HD + a.eps);
#pragma unroll
    for (int k = 0; k < PIECES; ++k) {
        const int i = lane + 32 * k;
        if (i < P) {
            const float4 wv = *reinterpret_cast<const float4*>(w + 4 * i);
            x[k][0] *= inv * wv.x; x[k][1] *= inv * wv.y; x[k][2] *= inv * wv.z; x[k][3] *= inv * wv.w;
        }
    }
    // partner piece of piece i inside the rotated part: i + hp (first half) or i - hp (second half)
#pragma unroll
    for (int k = 0; k < PIECES; ++k) {
        const int i = lane + 32 * k;
        const bool rot_lo = i < hp, rot_hi = !rot_lo && i < rp;
        const int pi = rot_lo ? i + hp : i - hp;                 // partner piece (meaningful when rotated)
        float px[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            // the partner's value: from lane pi % 32, its piece pi / 32 (every lane takes part in the shuffles)
            float v = 0.0f;
#pragma unroll
            for (int kk = 0; kk < PIECES; ++kk) {
                const float cand = __shfl_sync(0xffffffffu, x[kk][e], (rot_lo || rot_hi) ? (pi & 31) : lane);
                if ((rot_lo || rot_hi) && (pi >> 5) == kk) v = cand;
            }
            px[e] = v;
        }
        if (i < P) {
            float r[4];
            if (rot_lo || rot_hi) {
                const int t = rot_lo ? i : i - hp;               // table piece
                const float4 c = *reinterpret_cast<const float4*>(s_cos + 4 * t);
                const float4 sn = *reinterpret_cast<const float4*>(s_sin + 4 * t);
                if (rot_lo) {
                    r[0] = x[k][0] * c.x - px[0] * sn.x; r[1] = x[k][1] * c.y - px[1] * sn.y;
                    r[2] = x[k][2] * c.z - px[2] * sn.z; r[3] = x[k][3] * c.w - px[3] * sn.w;
                } else {
                    r[0] = px[0] * sn.x + x[k][0] * c.x; r[1] = px[1] * sn.y + x[k][1] * c.y;
                    r[2] = px[2] * sn.z + x[k][2] * c.z; r[3] = px[3] * sn.w + x[k][3] * c.w;
                }
            } else {
                r[0] = x[k][0]; r[1] = x[k][1]; r[2] = x[k][2]; r[3] = x[k][3];
            }
            uint2 o;
            o.x = pack_half2(r[0], r[1]);
            o.y = pack_half2(r[2], r[3]);
            reinterpret_cast<uint2*>(dst)[i] = o;
        }
    }
}

// Grid = (CTAs per token, tokens). A CTA takes every gridDim.x-th group of kRopeWarps units of its
// token: a unit is a query head, a key head or a value head (j < H query head j, j < H + KVH key
// head, else value head — a plain copy, only when a cache is given).
//   * The rotation angles depend on (position, pair index) only, so a CTA computes the cos/sin
//     table of its token once (rot/2 entries, accurate powf + sincosf: positions reach 10^5 rad)
//     and every head of the token reuses it — the reference recomputes it per head and per pair.
//   * `vec` (host: 8-byte aligned rows, head_dim and rotary_dim/2 multiples of 4): a head lives in
//     registers, 4 elements per lane and piece, partners reached by shuffles, 8-byte global accesses and
//     16-byte reads of the tables. Otherwise a warp stages its head as fp32 in shared memory and works
//     element by element, so any rotary_dim <= head_dim <= 512 and any alignment take the same kernel.
__global__ void __launch_bounds__(kRopeWarps * 32) hkv_qk_norm_rope_kernel(const RopeArgs a, const int vec) {
    __shared__ float s_x[kRopeWarps][512];
    __shared__ __align__(16) float s_cos[256];
    __shared__ __align__(16) float s_sin[256];
    __shared__ __align__(16) float s_w[2][512];          // q and k norm weights as fp32
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tok = a.H + 2 * a.KVH;
    const int half_rot = a.rot / 2;
    for (int i = threadIdx.x; i < a.HD; i += blockDim.x) {
        s_w[0][i] = __half2float(a.q_w[i]);
        s_w[1][i] = __half2float(a.k_w[i]);
    }
    const long long tokens = (long long)a.B * a.S;
    for (long long tok = blockIdx.y; tok < tokens; tok += gridDim.y) {
        const int s = (int)(tok % a.S), b = (int)(tok / a.S);
        const int pos = (a.d_pos ? a.d_pos[b * a.pos_stride] : a.host_pos) + s;
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
        int slot = -2;                      // row of this token in the cache planes, looked up once
        for (int j = blockIdx.x * kRopeWarps + warp; j < per_tok; j += gridDim.x * kRopeWarps) {
            const bool is_q = j < a.H, is_k = !is_q && j < a.H + a.KVH;
            const int kvh = is_q ? 0 : (is_k ? j - a.H : j - a.H - a.KVH);
            if (!is_q && a.k_cache) {
                if (slot == -2) slot = slot_of_pos(a.map, pos);
                if (slot < 0) continue;     // dropped past the plane / owned by another rank
            }
            const long long cache_off = (long long)b * a.batch_stride + ((long long)slot * a.KVH + kvh) * a.HD;
            if (!is_q && !is_k) {           // value head: plain copy into the cache
                if (!a.k_cache || !a.v) continue;
                const __half* src = a.v + ((tok * a.KVH) + kvh) * a.HD;
                __half* dst = a.v_cache + cache_off;
                if (vec) {
                    for (int i = lane; i < a.HD / 4; i += 32) reinterpret_cast<uint2*>(dst)[i] = reinterpret_cast<const uint2*>(src)[i];
                } else {
                    for (int i = lane; i < a.HD; i += 32) dst[i] = src[i];
                }
                continue;
            }
            const __half* src = is_q ? a.q + (tok * a.H + j) * a.HD : a.k + (tok * a.KVH + kvh) * a.HD;
            __half* dst = is_q ? a.q + (tok * a.H + j) * a.HD
                               : (a.k_cache ? a.k_cache + cache_off : a.k + (tok * a.KVH + kvh) * a.HD);
            const float* w = s_w[is_q ? 0 : 1];
            if (!vec) rope_unit_scalar(a, src, dst, w, half_rot, s_x[warp], s_cos, s_sin, lane);
            else if (a.HD <= 128) rope_unit_vec<1>(a, src, dst, w, half_rot, s_cos, s_sin, lane);
            else if (a.HD <= 256) rope_unit_vec<2>(a, src, dst, w, half_rot, s_cos, s_sin, lane);
            else rope_unit_vec<4>(a, src, dst, w, half_rot, s_cos, s_sin, lane);
        }
    }
}

}  // namespace hkv
