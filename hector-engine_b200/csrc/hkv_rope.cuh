// hkv_rope.cuh — per-head RMSNorm of q and k + rotary embedding, with the rotated K and the
// V row written straight into the cache planes (the front of the append path).
//
// Replaces qk_norm_rope_kernel<DEVICE_POS, WRITE_CACHE> and its launchers (reference
// kernels/attention.cu:800-973): same arithmetic
//   x_n[i] = x[i] * rsqrt(mean(x^2) + eps) * w[i]
//   pairs (i, i + rot/2), i < rot/2, rotated by ((s + pos) / scaling) / theta^(2i/rot)
//   dims >= rot pass through normalised
// but batched over sequences with one device position per sequence, row lookup through
// the same position->row map as the append (linear drop / ring / shard owner), a group of lanes per
// (sequence, token, head), the rotation table computed once per token and CTA, 16-byte accesses.
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

// The cos/sin table of one token: rot/2 entries, accurate powf + sincosf (positions reach 10^5 rad).
__device__ __forceinline__ void rope_fill_table(const RopeArgs& a, const int pos, const int half_rot, float* s_cos,
                                                float* s_sin) {
    const float fp = (float)pos / a.scaling;
    for (int i = threadIdx.x; i < half_rot; i += blockDim.x) {
        const float freq = 1.0f / powf(a.theta, (float)(2 * i) / (float)a.rot);
        float sn, c;
        sincosf(fp * freq, &sn, &c);
        s_cos[i] = c;
        s_sin[i] = sn;
    }
}

// Where unit j of token `tok` is read: a query head (j < H), a key head (j < H + KVH) or a value head.
__device__ __forceinline__ const __half* rope_unit_src(const RopeArgs& a, const long long tok, const int j) {
    if (j < a.H) return a.q + (tok * a.H + j) * a.HD;
    if (j < a.H + a.KVH) return a.k + (tok * a.KVH + (j - a.H)) * a.HD;
    return a.v + (tok * a.KVH + (j - a.H - a.KVH)) * a.HD;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&x)[8]) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&raw.z));
    const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&raw.w));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}

// The register path (host: rows 16-byte aligned, head_dim a multiple of 8 and at most 256, rotary_dim/2
// a multiple of 8). A head is held by the smallest power-of-two group of lanes that covers its 16-byte
// pieces (16 lanes for head_dim 128: a warp works on TWO heads at a time), one piece of 8 elements per
// lane. What keeps the instruction count per byte low — the first version of this kernel was bound by
// instruction issue, not by memory:
//   * the rotation partner of a piece is a whole piece rot/16 lanes away: its RAW 16 bytes come over in
//     four shuffles and are normalised here with the partner's weights (same head, same 1/rms);
//   * pieces outside the rotated span use cos = 1, sin = 0, query/key/value lanes differ only in the
//     weights they read and in the address they store to: no divergent branches in the unit;
//   * a CTA owns a contiguous range of tokens, computes theta^(-2i/rot) once, and the cos/sin tables of
//     up to four tokens at a time with all its threads (one sincosf per thread);
//   * every warp issues the 16-byte loads of U of its units before it touches the first.
template <int U>
__device__ __forceinline__ void rope_tokens_fast(const RopeArgs& a, float* s_cos, float* s_sin, float* s_freq,
                                                 float (*s_w)[512], int* s_row) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int half_rot = a.rot / 2;
    const int P = a.HD / 8, hp = half_rot / 8, rp = a.rot / 8;
    int LPH = 1;                                   // lanes per head
    while (LPH < P) LPH <<= 1;
    const int HPW = 32 / LPH;                      // heads per warp
    const int sub = lane / LPH, p = lane % LPH;
    const bool lane_live = p < P;
    const bool rot_lo = p < hp, rot_hi = !rot_lo && p < rp;
    const int pi = rot_lo ? p + hp : (rot_hi ? p - hp : p);     // partner piece
    const int src_lane = lane - p + pi;
    const int tpiece = rot_lo ? p : p - hp;                     // table piece (when rotated)
    const float sgn = rot_lo ? -1.0f : 1.0f;
    const bool copy_v = a.k_cache && a.v;
    const int per_tok = a.H + a.KVH + (copy_v ? a.KVH : 0);
    const int slots_per_tok = (per_tok + HPW - 1) / HPW;

    for (int i = tid; i < a.HD; i += blockDim.x) {
        s_w[0][i] = __half2float(a.q_w[i]);
        s_w[1][i] = __half2float(a.k_w[i]);
    }
    for (int i = tid; i < half_rot; i += blockDim.x) s_freq[i] = 1.0f / powf(a.theta, (float)(2 * i) / (float)a.rot);

    const long long tokens = (long long)a.B * a.S;
    const long long per = (tokens + gridDim.y - 1) / gridDim.y;
    const long long t_begin = blockIdx.y * per;
    const long long t_end = t_begin + per < tokens ? t_begin + per : tokens;
    int TB = (int)blockDim.x / (half_rot > 0 ? half_rot : 1);   // tokens whose tables fit one pass of the CTA
    TB = TB < 1 ? 1 : (TB > 4 ? 4 : TB);
    const int stride = gridDim.x * kRopeWarps;

    for (long long tb = t_begin; tb < t_end; tb += TB) {
        const int nb = (int)(t_end - tb < TB ? t_end - tb : TB);
        __syncthreads();                    // weights and frequencies written; the previous tables no longer read
        for (int e = tid; e < nb * half_rot; e += blockDim.x) {
            const int tt = e / half_rot, i = e - tt * half_rot;
            const long long tok = tb + tt;
            const int s = (int)(tok % a.S), b = (int)(tok / a.S);
            const int pos = (a.d_pos ? a.d_pos[b * a.pos_stride] : a.host_pos) + s;
            float sn, c;
            sincosf(((float)pos / a.scaling) * s_freq[i], &sn, &c);
            s_cos[e] = c;
            s_sin[e] = sn;
            if (i == 0) s_row[tt] = a.k_cache ? slot_of_pos(a.map, pos) : -1;
        }
        if (half_rot == 0) {
            for (int tt = tid; tt < nb; tt += blockDim.x) {
                const long long tok = tb + tt;
                const int pos = (a.d_pos ? a.d_pos[(int)(tok / a.S) * a.pos_stride] : a.host_pos) + (int)(tok % a.S);
                s_row[tt] = a.k_cache ? slot_of_pos(a.map, pos) : -1;
            }
        }
        __syncthreads();
        const int items = nb * slots_per_tok;
        for (int it0 = blockIdx.x * kRopeWarps + warp; it0 < items; it0 += U * stride) {
            uint4 raw[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int it = it0 + u * stride;
                const int tt = it / slots_per_tok, j = (it - tt * slots_per_tok) * HPW + sub;
                const bool ok = it < items && lane_live && j < per_tok;
                raw[u] = ok ? __ldg(reinterpret_cast<const uint4*>(rope_unit_src(a, tb + tt, j)) + p)
                            : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int it = it0 + u * stride;
                if (it >= items) break;     // warp-uniform
                const int tt = it / slots_per_tok, j = (it - tt * slots_per_tok) * HPW + sub;
                const long long tok = tb + tt;
                const bool is_q = j < a.H, is_k = !is_q && j < a.H + a.KVH;
                float x[8], px[8];
                unpack8(raw[u], x);
                float ssq = 0.0f;
#pragma unroll
                for (int e = 0; e < 8; ++e) ssq = fmaf(x[e], x[e], ssq);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
                    if (o < LPH) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
                const float inv = 1.0f / sqrtf(ssq / (float)a.HD + a.eps);
                uint4 praw;
                praw.x = __shfl_sync(0xffffffffu, raw[u].x, src_lane);
                praw.y = __shfl_sync(0xffffffffu, raw[u].y, src_lane);
                praw.z = __shfl_sync(0xffffffffu, raw[u].z, src_lane);
                praw.w = __shfl_sync(0xffffffffu, raw[u].w, src_lane);
                unpack8(praw, px);
                if (!lane_live || j >= per_tok) continue;
                const float* w = s_w[is_q ? 0 : 1];
                const bool rotated = rot_lo || rot_hi;
                const float* tc = s_cos + tt * half_rot + 8 * tpiece;
                const float* ts = s_sin + tt * half_rot + 8 * tpiece;
                uint32_t packed[4];
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {      // four elements at a time: fewer live registers
                    const float4 wn = *reinterpret_cast<const float4*>(w + 8 * p + 4 * hf);
                    const float4 wp = *reinterpret_cast<const float4*>(w + 8 * pi + 4 * hf);
                    float4 cc = make_float4(1.f, 1.f, 1.f, 1.f), ss = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (rotated) {
                        cc = *reinterpret_cast<const float4*>(tc + 4 * hf);
                        ss = *reinterpret_cast<const float4*>(ts + 4 * hf);
                    }
                    const float* xs = x + 4 * hf;
                    const float* ps = px + 4 * hf;
                    const float r0 = fmaf(sgn * (ps[0] * (inv * wp.x)), ss.x, (xs[0] * (inv * wn.x)) * cc.x);
                    const float r1 = fmaf(sgn * (ps[1] * (inv * wp.y)), ss.y, (xs[1] * (inv * wn.y)) * cc.y);
                    const float r2 = fmaf(sgn * (ps[2] * (inv * wp.z)), ss.z, (xs[2] * (inv * wn.z)) * cc.z);
                    const float r3 = fmaf(sgn * (ps[3] * (inv * wp.w)), ss.w, (xs[3] * (inv * wn.w)) * cc.w);
                    packed[2 * hf] = pack_half2(r0, r1);
                    packed[2 * hf + 1] = pack_half2(r2, r3);
                }
                uint4 o = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                __half* dst;
                if (is_q) {
                    dst = a.q + (tok * a.H + j) * a.HD;
                } else {
                    const int kvh = is_k ? j - a.H : j - a.H - a.KVH;
                    if (a.k_cache) {
                        const int row = s_row[tt];
                        if (row < 0) continue;          // dropped past the plane / owned by another rank
                        const long long off = (tok / a.S) * a.batch_stride + ((long long)row * a.KVH + kvh) * a.HD;
                        dst = (is_k ? a.k_cache : a.v_cache) + off;
                        if (!is_k) o = raw[u];          // value head: plain copy into the cache
                    } else {
                        dst = a.k + (tok * a.KVH + kvh) * a.HD;
                    }
                }
                reinterpret_cast<uint4*>(dst)[p] = o;
            }
        }
    }
}

// Grid = (CTAs per token range, token ranges): CTA (x, y) takes the y-th contiguous range of tokens and,
// of its units, every gridDim.x-th group of kRopeWarps. A unit is a query head, a key head or a value
// head (j < H query head j, j < H + KVH key head, else value head — a plain copy, only when a cache
// is given).
//   * The rotation angles depend on (position, pair index) only, so a CTA computes the cos/sin table of
//     a token once and every head of the token reuses it — the reference recomputes it per head and
//     per pair.
//   * `fast`: the register path above. Otherwise a warp stages one head as fp32 in shared memory and
//     works element by element, so any rotary_dim <= head_dim <= 512 and any alignment take the same
//     kernel.
__global__ void __launch_bounds__(kRopeWarps * 32, 4) hkv_qk_norm_rope_kernel(const RopeArgs a, const int fast) {
    __shared__ __align__(16) float s_cos[256];
    __shared__ __align__(16) float s_sin[256];
    __shared__ __align__(16) float s_w[2][512];          // q and k norm weights as fp32
    if (fast) {
        __shared__ float s_freq[256];
        __shared__ int s_row[4];
        rope_tokens_fast<3>(a, s_cos, s_sin, s_freq, s_w, s_row);
        return;
    }
    __shared__ float s_x[kRopeWarps][512];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tok = a.H + 2 * a.KVH;
    const int half_rot = a.rot / 2;
    for (int i = threadIdx.x; i < a.HD; i += blockDim.x) {
        s_w[0][i] = __half2float(a.q_w[i]);
        s_w[1][i] = __half2float(a.k_w[i]);
    }
    const long long tokens = (long long)a.B * a.S;
    const long long per = (tokens + gridDim.y - 1) / gridDim.y;
    const long long t_begin = blockIdx.y * per;
    const long long t_end = t_begin + per < tokens ? t_begin + per : tokens;
    for (long long tok = t_begin; tok < t_end; ++tok) {
        const int s = (int)(tok % a.S), b = (int)(tok / a.S);
        const int pos = (a.d_pos ? a.d_pos[b * a.pos_stride] : a.host_pos) + s;
        __syncthreads();                    // the previous token's table is no longer being read
        rope_fill_table(a, pos, half_rot, s_cos, s_sin);
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
                for (int i = lane; i < a.HD; i += 32) dst[i] = src[i];
                continue;
            }
            const __half* src = rope_unit_src(a, tok, j);
            __half* dst = is_q ? a.q + (tok * a.H + j) * a.HD
                               : (a.k_cache ? a.k_cache + cache_off : a.k + (tok * a.KVH + kvh) * a.HD);
            rope_unit_scalar(a, src, dst, s_w[is_q ? 0 : 1], half_rot, s_x[warp], s_cos, s_sin, lane);
        }
    }
}

}  // namespace hkv
