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
// lane. The kernel moves 256-byte rows and must stay under ~0.15 warp instructions per byte to be
// bound by memory rather than by instruction issue (its first versions were not), so:
//   * a CTA owns a contiguous range of tokens, computes theta^(-2i/rot) once and, for up to four
//     tokens at a time, the cos/sin of each pair with all its threads (one sincosf per thread), then
//     folds them with the norm weights into two tables per (token, q|k):
//         A[i] = w[i]·cos_i   B[i] = ∓w[partner(i)]·sin_i     (A = w, B = 0 outside the rotated span)
//     so that an output element is  rsqrt(mean(x²)+eps) · (x[i]·A[i] + x[partner(i)]·B[i]):
//     three floating-point instructions, no branch, the same code for every lane;
//   * the partner of a piece is a whole piece rot/16 lanes away: its RAW 16 bytes come over in four
//     shuffles; query / key / value lanes differ only in table and store address;
//   * (token, unit) pairs are walked incrementally — no division in the loop — and every warp issues
//     the 16-byte loads of U of its units before it touches the first.
template <int U>
__device__ __forceinline__ void rope_tokens_fast(const RopeArgs& a, float* s_cos, float* s_sin, float* s_freq,
                                                 float (*s_w)[512], float* s_A, float* s_B, long long* s_off) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int HD = a.HD, half_rot = a.rot / 2;
    const int P = HD / 8, hp = half_rot / 8, rp = a.rot / 8;
    int LPH = 1;                                   // lanes per head
    while (LPH < P) LPH <<= 1;
    const int HPW = 32 / LPH;                      // heads per warp
    const int sub = lane / LPH, p = lane % LPH;
    const bool lane_live = p < P;
    const bool rot_lo = p < hp, rot_hi = !rot_lo && p < rp;
    const int pi = rot_lo ? p + hp : (rot_hi ? p - hp : p);     // partner piece
    const int src_lane = lane - p + pi;
    const bool copy_v = a.k_cache && a.v;
    const int HK = a.H + a.KVH;
    const int per_tok = HK + (copy_v ? a.KVH : 0);
    const int spt = (per_tok + HPW - 1) / HPW;     // warp-level units ("slots") per token
    const float inv_hd = 1.0f / (float)HD;

    for (int i = tid; i < HD; i += blockDim.x) {
        s_w[0][i] = __half2float(a.q_w[i]);
        s_w[1][i] = __half2float(a.k_w[i]);
    }
    for (int i = tid; i < half_rot; i += blockDim.x) s_freq[i] = 1.0f / powf(a.theta, (float)(2 * i) / (float)a.rot);

    const long long tokens = (long long)a.B * a.S;
    const long long per = (tokens + gridDim.y - 1) / gridDim.y;
    const long long t_begin = blockIdx.y * per;
    const long long t_end = t_begin + per < tokens ? t_begin + per : tokens;
    int TB = (int)blockDim.x / (half_rot > 0 ? half_rot : 1);   // tokens whose angles fit one pass of the CTA
    TB = TB < 1 ? 1 : (TB > 4 ? 4 : TB);
    const int stride = gridDim.x * kRopeWarps;

    for (long long tb = t_begin; tb < t_end; tb += TB) {
        const int nb = (int)(t_end - tb < TB ? t_end - tb : TB);
        const __half* q_base = a.q + tb * a.H * HD + 8 * p;
        const __half* k_base = a.k + tb * a.KVH * HD + 8 * p;
        const __half* v_base = copy_v ? a.v + tb * a.KVH * HD + 8 * p : nullptr;
        int it = blockIdx.x * kRopeWarps + warp;
        int tt = it / spt, slot = it - tt * spt;
        uint4 raw[U];
        int utt[U], uj[U];
        const __half* usrc[U];
        // Issues the loads of this warp's next U units (they need nothing but the token index).
        auto load_round = [&]() {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                utt[u] = tt;
                uj[u] = slot * HPW + sub;
                const int j = uj[u];
                const bool ok = tt < nb && lane_live && j < per_tok;
                const __half* src = j < a.H ? q_base + (tt * a.H + j) * HD
                                  : j < HK  ? k_base + (tt * a.KVH + (j - a.H)) * HD
                                            : v_base + (tt * a.KVH + (j - HK)) * HD;
                raw[u] = ok ? __ldg(reinterpret_cast<const uint4*>(src)) : make_uint4(0u, 0u, 0u, 0u);
                usrc[u] = src;
                slot += stride;
                while (slot >= spt) { slot -= spt; ++tt; }
            }
        };
        // The first round's rows and this thread's position are requested BEFORE the tables are built:
        // their latency runs under the trigonometry (a decode-sized launch is nothing but these latencies).
        load_round();
        int pos_pre = 0;
        if (tid < nb * half_rot) {
            const long long tok = tb + tid / half_rot;
            pos_pre = (a.d_pos ? a.d_pos[(int)(tok / a.S) * a.pos_stride] : a.host_pos) + (int)(tok % a.S);
        }
        __syncthreads();                    // weights and frequencies written; the previous tables no longer read
        for (int e = tid; e < nb * half_rot; e += blockDim.x) {
            const int t = e / half_rot, i = e - t * half_rot;
            const long long tok = tb + t;
            const int pos = e == tid ? pos_pre
                                     : (a.d_pos ? a.d_pos[(int)(tok / a.S) * a.pos_stride] : a.host_pos) + (int)(tok % a.S);
            float sn, c;
            sincosf(((float)pos / a.scaling) * s_freq[i], &sn, &c);
            s_cos[e] = c;
            s_sin[e] = sn;
        }
        if (tid < nb) {                     // where the token's K/V rows go: element offset into the planes, or -1
            const long long tok = tb + tid;
            const int b = (int)(tok / a.S);
            const int pos = (a.d_pos ? a.d_pos[b * a.pos_stride] : a.host_pos) + (int)(tok % a.S);
            const int row = a.k_cache ? slot_of_pos(a.map, pos) : -1;
            s_off[tid] = row < 0 ? -1 : (long long)b * a.batch_stride + (long long)row * a.KVH * HD;
        }
        __syncthreads();
        for (int t = 0; t < nb; ++t) {      // the folded tables of token t: [q | k][HD]
            const float* cs = s_cos + t * half_rot;
            const float* sn = s_sin + t * half_rot;
            for (int r = tid; r < 2 * HD; r += blockDim.x) {
                const int kind = r >= HD ? 1 : 0, i = r - kind * HD;
                const float* w = s_w[kind];
                float A = w[i], B = 0.0f;
                if (i < half_rot) {
                    A *= cs[i];
                    B = -w[i + half_rot] * sn[i];
                } else if (i < a.rot) {
                    A *= cs[i - half_rot];
                    B = w[i - half_rot] * sn[i - half_rot];
                }
                s_A[t * 2 * HD + r] = A;
                s_B[t * 2 * HD + r] = B;
            }
        }
        __syncthreads();
        while (utt[0] < nb) {               // warp-uniform
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (utt[u] >= nb) break;    // warp-uniform
                const int j = uj[u], t = utt[u];
                float x[8], px[8];
                unpack8(raw[u], x);
                float ssq = 0.0f;
#pragma unroll
                for (int e = 0; e < 8; ++e) ssq = fmaf(x[e], x[e], ssq);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
                    if (o < LPH) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
                const float inv = rsqrtf(fmaf(ssq, inv_hd, a.eps));
                uint4 praw;
                praw.x = __shfl_sync(0xffffffffu, raw[u].x, src_lane);
                praw.y = __shfl_sync(0xffffffffu, raw[u].y, src_lane);
                praw.z = __shfl_sync(0xffffffffu, raw[u].z, src_lane);
                praw.w = __shfl_sync(0xffffffffu, raw[u].w, src_lane);
                if (!lane_live || j >= per_tok) continue;
                const bool is_q = j < a.H;
                uint4 o;
                if (j < HK) {
                    unpack8(praw, px);
                    const float* tA = s_A + ((t * 2 + (is_q ? 0 : 1)) * HD + 8 * p);
                    const float* tB = s_B + ((t * 2 + (is_q ? 0 : 1)) * HD + 8 * p);
                    const float4 a0 = *reinterpret_cast<const float4*>(tA), a1 = *reinterpret_cast<const float4*>(tA + 4);
                    const float4 b0 = *reinterpret_cast<const float4*>(tB), b1 = *reinterpret_cast<const float4*>(tB + 4);
                    o.x = pack_half2(inv * fmaf(px[0], b0.x, x[0] * a0.x), inv * fmaf(px[1], b0.y, x[1] * a0.y));
                    o.y = pack_half2(inv * fmaf(px[2], b0.z, x[2] * a0.z), inv * fmaf(px[3], b0.w, x[3] * a0.w));
                    o.z = pack_half2(inv * fmaf(px[4], b1.x, x[4] * a1.x), inv * fmaf(px[5], b1.y, x[5] * a1.y));
                    o.w = pack_half2(inv * fmaf(px[6], b1.z, x[6] * a1.z), inv * fmaf(px[7], b1.w, x[7] * a1.w));
                } else {
                    o = raw[u];             // value head: plain copy into the cache
                }
                __half* dst;
                if (is_q) {
                    dst = const_cast<__half*>(usrc[u]);      // rewritten in place
                } else {
                    const int kvh = j < HK ? j - a.H : j - HK;
                    if (a.k_cache) {
                        const long long off = s_off[t];
                        if (off < 0) continue;          // dropped past the plane / owned by another rank
                        dst = (j < HK ? a.k_cache : a.v_cache) + off + kvh * HD + 8 * p;
                    } else {
                        dst = const_cast<__half*>(usrc[u]);  // no cache: k rewritten in place
                    }
                }
                *reinterpret_cast<uint4*>(dst) = o;
            }
            if (tt >= nb) break;            // warp-uniform: nothing left for this warp in the stage
            load_round();
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
    __shared__ __align__(16) float s_buf[kRopeWarps * 512];   // fast: the A and B tables; else: the warps' staging rows
    if (fast) {
        __shared__ float s_freq[256];
        __shared__ long long s_off[4];
        rope_tokens_fast<3>(a, s_cos, s_sin, s_freq, s_w, s_buf, s_buf + 2048, s_off);
        return;
    }
    float (*s_x)[512] = reinterpret_cast<float (*)[512]>(s_buf);
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
