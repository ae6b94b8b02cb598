// hkv_oracle.cpp — CPU oracle for the KV-append + cached-attention path.
//
// TEST INFRASTRUCTURE ONLY. This file is the checker, never the product: only the
// test-suite, the smoke check and the benchmark's CPU-baseline leg may load it.
// The shipped library (libhkv) contains no CPU path and never links this file.
//
// It restates, as scalar C++ with fp32 accumulation, the semantics of the
// reference's CUDA kernels (paths are relative to the reference project root):
//   append            kernels/attention.cu:1119-1151  (kv_cache_update_kernel_dp)
//   decode attention  kernels/attention.cu:337-494    (attention_cached_v2_kernel_dp)
//   prefill-cached    kernels/attention.cu:664-773    (attention_prefill_cached_kernel)
//   op defaults       kernels/register_kernels.cpp:851-861, src/command.cpp:160
//   cache layouts     src/kv_cache.hpp:175-199, src/gemma4_kv_cache.hpp:39-114
//   QK-norm + RoPE    kernels/attention.cu:800-906 (with K/V cache write: :947-973)
//
// Parity pinning: the known-answer cases of the reference's own hot-path test
// (tests/test_gemma4_kv.cu:110-347) are replayed against this file by the CPU test
// suite, and golden vectors produced by the reference kernels themselves (rebuilt for
// sm_100a and run on a B200) are compared against it as committed fixtures.
//
// The grading oracle ("exact" mode) is a position-ordered two-pass softmax with fp32
// accumulation and an accurate expf. A second mode ("ref16") reproduces the
// reference's order of operations (16 contiguous chunks, online softmax inside each,
// -1e10f start value, merge through a global maximum) and exists only to diagnose
// differences between the two.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

// ---------------------------------------------------------------------------
// IEEE binary16 <-> binary32, round-to-nearest-even (what __float2half and
// __floats2half2_rn do, kernels/attention.cu:312, :488-490).
// ---------------------------------------------------------------------------
inline float h2f(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: normalise
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t f2h(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u : 0u));
    }
    if (x >= 0x477FF000u) {  // rounds to >= 65520 -> inf
        return (uint16_t)(sign | 0x7C00u);
    }
    if (x < 0x38800000u) {  // result is subnormal or zero (|f| < 2^-14)
        if (x < 0x33000000u) return (uint16_t)sign;  // < 2^-25 -> 0
        const int e = (int)(x >> 23);                // biased fp32 exponent
        uint32_t man = (x & 0x7FFFFFu) | 0x800000u;  // 24-bit significand
        const int shift = 126 - e;                   // 14..24
        const uint32_t half_man = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1u);
        const uint32_t halfway = 1u << (shift - 1);
        uint32_t r = half_man;
        if (rem > halfway || (rem == halfway && (half_man & 1u))) ++r;
        return (uint16_t)(sign | r);
    }
    uint32_t man = x & 0x7FFFFFu;
    uint32_t e = (x >> 23) - 112u;
    uint32_t r = (e << 10) | (man >> 13);
    const uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;  // carries into exponent correctly
    return (uint16_t)(sign | r);
}

// ---------------------------------------------------------------------------
// Counter-based synthetic data: identical bits on CPU and GPU.
// value(seed, i) = (2*sum12 - 786420) * 2^-17 where sum12 is the sum of twelve
// 16-bit uniform fields of three splitmix64 outputs (Irwin-Hall(12): mean 0,
// variance 1 to 2e-10, support +-6). Every step is exact in fp32, so the CUDA
// twin of this function produces the same fp16 bit pattern.
// ---------------------------------------------------------------------------
inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

inline uint16_t synth_half(uint64_t seed, uint64_t i) {
    const uint64_t base = splitmix64(seed ^ (i * 0xD1342543DE82EF95ull));
    uint32_t sum = 0;
    for (int r = 0; r < 3; ++r) {
        const uint64_t v = splitmix64(base + (uint64_t)r);
        sum += (uint32_t)(v & 0xFFFF) + (uint32_t)((v >> 16) & 0xFFFF) +
               (uint32_t)((v >> 32) & 0xFFFF) + (uint32_t)((v >> 48) & 0xFFFF);
    }
    const float x = (float)((int32_t)(2u * sum) - 786420) * (1.0f / 131072.0f);
    return f2h(x);
}

// Slot of logical position p in a plane with `slots` rows (layout 1 = ring).
inline int64_t slot_of(int64_t p, int slots, int layout) {
    return layout == 1 ? (p % slots) : p;
}

struct AttnGeom {
    int H, KVH, HD, slots, window, layout;
    int64_t batch_stride;  // elements between sequences in a cache plane
    float scale;
};

// One (sequence, query head): attend logical positions [first, total).
// Two-pass softmax, fp32 accumulation, position order.
void attend_exact(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, uint16_t* out,
                  float* out_f32, int total, const AttnGeom& g, int h) {
    const int G = g.H / g.KVH;
    const int kvh = (g.KVH == g.H) ? h : h / G;  // kernels/attention.cu:362
    int lim = total;
    if (g.layout == 0 && lim > g.slots) lim = g.slots;  // never read past the plane
    int first = g.window > 0 ? std::max(0, total - g.window) : 0;  // :385
    if (g.layout == 1) first = std::max(first, total - g.slots);   // ring keeps `slots` rows
    const int n = lim - first;
    std::vector<float> acc((size_t)g.HD, 0.0f);
    if (n <= 0) {  // seq_len 0 -> zero output (:478)
        for (int d = 0; d < g.HD; ++d) { out[d] = 0; if (out_f32) out_f32[d] = 0.0f; }
        return;
    }
    std::vector<float> qf((size_t)g.HD), s((size_t)n);
    for (int d = 0; d < g.HD; ++d) qf[d] = h2f(q[d]);
    float mx = -INFINITY;
    for (int i = 0; i < n; ++i) {
        const int64_t row = slot_of(first + i, g.slots, g.layout);
        const uint16_t* kr = kc + row * (int64_t)g.KVH * g.HD + (int64_t)kvh * g.HD;
        float dot = 0.0f;
        for (int d = 0; d < g.HD; ++d) dot = std::fmaf(qf[d], h2f(kr[d]), dot);
        s[i] = dot * g.scale;  // :416
        mx = std::max(mx, s[i]);
    }
    float l = 0.0f;
    for (int i = 0; i < n; ++i) {
        const float p = std::exp(s[i] - mx);
        l += p;
        const int64_t row = slot_of(first + i, g.slots, g.layout);
        const uint16_t* vr = vc + row * (int64_t)g.KVH * g.HD + (int64_t)kvh * g.HD;
        for (int d = 0; d < g.HD; ++d) acc[d] = std::fmaf(p, h2f(vr[d]), acc[d]);
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    for (int d = 0; d < g.HD; ++d) {
        const float o = acc[d] * inv;
        out[d] = f2h(o);
        if (out_f32) out_f32[d] = o;
    }
}

// Same (sequence, head) in the reference's operation order: 16 contiguous chunks,
// online softmax with -1e10f start, merge by global max (kernels/attention.cu:385-478).
void attend_ref16(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, uint16_t* out,
                  int total, const AttnGeom& g, int h) {
    const int W = 16;
    const int G = g.H / g.KVH;
    const int kvh = (g.KVH == g.H) ? h : h / G;
    const int first = g.window > 0 ? std::max(0, total - g.window) : 0;
    const int active = total - first;
    const int chunk = (active + W - 1) / W;
    std::vector<float> qf((size_t)g.HD);
    for (int d = 0; d < g.HD; ++d) qf[d] = h2f(q[d]);
    std::vector<float> pm(W), ps(W);
    std::vector<std::vector<float>> pa(W, std::vector<float>((size_t)g.HD, 0.0f));
    for (int w = 0; w < W; ++w) {
        float rmax = -1e10f, rsum = 0.0f;
        const int p0 = first + w * chunk, p1 = std::min(p0 + chunk, total);
        for (int pos = p0; pos < p1; ++pos) {
            const int64_t row = slot_of(pos, g.slots, g.layout);
            const uint16_t* kr = kc + row * (int64_t)g.KVH * g.HD + (int64_t)kvh * g.HD;
            const uint16_t* vr = vc + row * (int64_t)g.KVH * g.HD + (int64_t)kvh * g.HD;
            float dot = 0.0f;
            for (int d = 0; d < g.HD; ++d) dot = std::fmaf(qf[d], h2f(kr[d]), dot);
            const float score = dot * g.scale;
            const float nmax = std::max(rmax, score);
            const float e = std::exp(score - nmax), corr = std::exp(rmax - nmax);
            rsum = rsum * corr + e;
            for (int d = 0; d < g.HD; ++d) pa[w][d] = std::fmaf(e, h2f(vr[d]), pa[w][d] * corr);
            rmax = nmax;
        }
        pm[w] = rmax;
        ps[w] = rsum;
    }
    float gmax = pm[0];
    for (int w = 1; w < W; ++w) gmax = std::max(gmax, pm[w]);
    float msum = 0.0f;
    std::vector<float> macc((size_t)g.HD, 0.0f);
    for (int w = 0; w < W; ++w) {
        const float corr = std::exp(pm[w] - gmax);
        msum += ps[w] * corr;
        for (int d = 0; d < g.HD; ++d) macc[d] += pa[w][d] * corr;
    }
    const float inv = msum > 0.0f ? 1.0f / msum : 0.0f;
    for (int d = 0; d < g.HD; ++d) out[d] = f2h(macc[d] * inv);
}

template <class F>
void parallel_for(int n, int threads, F&& fn) {
    if (threads <= 1 || n <= 1) {
        for (int i = 0; i < n; ++i) fn(i);
        return;
    }
    std::atomic<int> next{0};
    std::vector<std::thread> pool;
    const int nt = std::min(threads, n);
    for (int t = 0; t < nt; ++t) {
        pool.emplace_back([&] {
            for (;;) {
                const int i = next.fetch_add(1);
                if (i >= n) break;
                fn(i);
            }
        });
    }
    for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

int hkv_oracle_abi_version() { return 1; }

int hkv_oracle_hardware_threads() {
    const unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}

uint16_t hkv_oracle_f2h(float f) { return f2h(f); }
float hkv_oracle_h2f(uint16_t h) { return h2f(h); }

// dst[i] = synthetic fp16 value for global element index (first_index + i).
void hkv_oracle_fill(uint16_t* dst, uint64_t seed, uint64_t first_index, uint64_t count) {
    for (uint64_t i = 0; i < count; ++i) dst[i] = synth_half(seed, first_index + i);
}

// KV append. new_k/new_v: [B, S, KVH, HD]; planes: [B, slots, KVH, HD] with
// `batch_stride` elements between sequences (0 = slots*KVH*HD). pos[b] is the write
// index of token 0 of sequence b. layout 0: row = pos+s, dropped when >= slots
// (kernels/attention.cu:1143-1148). layout 1 (ring, not in the reference): row = (pos+s) % slots.
void hkv_oracle_append(const uint16_t* new_k, const uint16_t* new_v, uint16_t* k_cache,
                       uint16_t* v_cache, int B, int S, int KVH, int HD, int slots,
                       int64_t batch_stride, const int32_t* pos, int layout) {
    const int64_t row = (int64_t)KVH * HD;
    if (batch_stride == 0) batch_stride = (int64_t)slots * row;
    for (int b = 0; b < B; ++b) {
        for (int s = 0; s < S; ++s) {
            int64_t p = (int64_t)pos[b] + s;
            if (p < 0) continue;
            if (layout == 1) p %= slots;
            else if (p >= slots) continue;
            const int64_t src = ((int64_t)b * S + s) * row;
            const int64_t dst = (int64_t)b * batch_stride + p * row;
            std::memcpy(k_cache + dst, new_k + src, (size_t)row * 2);
            std::memcpy(v_cache + dst, new_v + src, (size_t)row * 2);
        }
    }
}

// Decode attention. q/out: [B, 1, H, HD]; total[b] = attended length (cache_pos+1).
// mode 0 = exact oracle, 1 = reference operation order. out_f32 may be null.
void hkv_oracle_decode(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                       uint16_t* out, float* out_f32, int B, const int32_t* total, int H,
                       int KVH, int HD, int slots, int64_t batch_stride, float scale,
                       int window, int layout, int mode, int threads) {
    AttnGeom g{H, KVH, HD, slots, window, layout,
               batch_stride ? batch_stride : (int64_t)slots * KVH * HD, scale};
    parallel_for(B * H, threads, [&](int i) {
        const int b = i / H, h = i % H;
        const uint16_t* qp = q + ((int64_t)b * H + h) * HD;
        const uint16_t* kc = k_cache + (int64_t)b * g.batch_stride;
        const uint16_t* vc = v_cache + (int64_t)b * g.batch_stride;
        uint16_t* op = out + ((int64_t)b * H + h) * HD;
        if (mode == 1) attend_ref16(qp, kc, vc, op, total[b], g, h);
        else attend_exact(qp, kc, vc, op, out_f32 ? out_f32 + ((int64_t)b * H + h) * HD : nullptr,
                          total[b], g, h);
    });
}

// Prefill over the cache, batch 1 (kernels/attention.cu:664-773). q/out: [S_new, H, HD].
// Query i attends [first_i, past_len+i], first_i = window>0 ? max(0, past_len+i+1-window) : 0.
// q_begin/q_end select a sub-range of queries (for sampling long chunks).
void hkv_oracle_prefill(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                        uint16_t* out, float* out_f32, int S_new, int past_len, int H, int KVH,
                        int HD, int slots, float scale, int window, int q_begin, int q_end,
                        int threads) {
    AttnGeom g{H, KVH, HD, slots, window, 0, (int64_t)slots * KVH * HD, scale};
    if (q_end > S_new) q_end = S_new;
    const int nq = q_end - q_begin;
    if (nq <= 0) return;
    parallel_for(nq * H, threads, [&](int i) {
        const int qi = q_begin + i / H, h = i % H;
        const int64_t o = ((int64_t)qi * H + h) * HD;
        attend_exact(q + o, k_cache, v_cache, out + o, out_f32 ? out_f32 + o : nullptr,
                     past_len + qi + 1, g, h);
    });
}

// Fused per-head RMSNorm(q, k) + RoPE with optional K/V cache write
// (kernels/attention.cu:800-906, launcher :947-973). q: [B, S, H, HD] in place. k: [B, S, KVH, HD]:
// with a cache the normalised + rotated K goes to the cache row pos[b] + s (k itself untouched)
// and v is copied beside it; without a cache (k_cache null) k is rewritten in place.
// x_norm[i] = x[i] * rsqrt(mean(x^2) + eps) * w[i]; pairs (i, i + rot/2) for i < rot/2 are rotated
// by angle = ((s + pos) / scaling) / theta^(2i/rot); dims >= rot pass through normalised.
// Rows whose position falls outside the plane are dropped (layout 0) or wrap (layout 1).
void hkv_oracle_qk_norm_rope(uint16_t* q, uint16_t* k, const uint16_t* v, const uint16_t* q_w,
                             const uint16_t* k_w, uint16_t* k_cache, uint16_t* v_cache, int B, int S,
                             int H, int KVH, int HD, int rotary_dim, const int32_t* pos, int slots,
                             int layout, float eps, float theta, float scaling) {
    if (rotary_dim <= 0) rotary_dim = HD;
    if (scaling <= 0.0f) scaling = 1.0f;
    const int half_rot = rotary_dim / 2;
    std::vector<float> x((size_t)HD), y((size_t)HD);
    auto one = [&](const uint16_t* src, uint16_t* dst, const uint16_t* w, int p) {
        float ssq = 0.0f;
        for (int i = 0; i < HD; ++i) { x[i] = h2f(src[i]); ssq += x[i] * x[i]; }
        const float inv = 1.0f / std::sqrt(ssq / (float)HD + eps);
        for (int i = 0; i < HD; ++i) x[i] = x[i] * inv * h2f(w[i]);
        const float fp = (float)p / scaling;
        for (int i = 0; i < HD; ++i) y[i] = x[i];
        for (int i = 0; i < half_rot; ++i) {
            const float freq = 1.0f / std::pow(theta, (float)(2 * i) / (float)rotary_dim);
            const float ang = fp * freq;
            const float c = std::cos(ang), sn = std::sin(ang);
            y[i] = x[i] * c - x[i + half_rot] * sn;
            y[i + half_rot] = x[i] * sn + x[i + half_rot] * c;
        }
        for (int i = 0; i < HD; ++i) dst[i] = f2h(y[i]);
    };
    for (int b = 0; b < B; ++b)
        for (int s = 0; s < S; ++s) {
            const int p = pos[b] + s;
            for (int h = 0; h < H; ++h) {
                uint16_t* qp = q + (((int64_t)b * S + s) * H + h) * HD;
                one(qp, qp, q_w, p);
            }
            int64_t row = p;
            bool stored = true;
            if (k_cache) {
                if (layout == 1) row = p % slots;
                else if (p >= slots || p < 0) stored = false;
            }
            for (int h = 0; h < KVH; ++h) {
                uint16_t* kp = k + (((int64_t)b * S + s) * KVH + h) * HD;
                if (!k_cache) { one(kp, kp, k_w, p); continue; }
                if (!stored) continue;
                const int64_t dst = (((int64_t)b * slots + row) * KVH + h) * HD;
                one(kp, k_cache + dst, k_w, p);
                std::memcpy(v_cache + dst, v + (((int64_t)b * S + s) * KVH + h) * HD, (size_t)HD * 2);
            }
        }
}

// Heterogeneous / shared KV layout (src/gemma4_kv_cache.hpp:39-114). Inputs per layer:
// head_dim[i], is_global[i]. The first (layers - shared) layers own slots laid out back to
// back, each B*slots_i*KVH*head_dim[i] elements; later layers alias the last local / last
// global owner. ring_window > 0 gives local owners ring planes of `ring_window` rows
// (not in the reference, which keeps max_seq rows for every layer). Outputs: source[i],
// offset_elems[i], rows[i]. Returns elements per plane, or -1 for an invalid layout.
int64_t hkv_oracle_gemma4_layout(int layers, int shared, const int32_t* head_dim,
                                 const int32_t* is_global, int KVH, int B, int max_seq,
                                 int ring_window, int32_t* source, int64_t* offset_elems,
                                 int32_t* rows) {
    if (layers <= 0 || shared > layers || KVH <= 0 || B <= 0 || max_seq <= 0) return -1;
    const int first_shared = layers - shared;
    if (first_shared == 0) return -1;
    int last_local = -1, last_global = -1;
    int64_t total = 0;
    for (int i = 0; i < first_shared; ++i) {
        if (head_dim[i] <= 0) return -1;
        source[i] = i;
        offset_elems[i] = total;
        rows[i] = (!is_global[i] && ring_window > 0) ? std::min(ring_window, max_seq) : max_seq;
        if (is_global[i]) last_global = i; else last_local = i;
        total += (int64_t)B * rows[i] * KVH * head_dim[i];
    }
    for (int i = first_shared; i < layers; ++i) {
        const int src = is_global[i] ? last_global : last_local;
        if (src < 0 || head_dim[i] != head_dim[src]) return -1;
        source[i] = src;
        offset_elems[i] = offset_elems[src];
        rows[i] = rows[src];
    }
    return total;
}

}  // extern "C"
