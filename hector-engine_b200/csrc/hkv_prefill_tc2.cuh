// hkv_prefill_tc2.cuh — the tensor-core prefill kernel with TWO query tiles in flight per CTA.
//
// Same contract as hkv_prefill_tc_kernel (reference kernels/attention.cu:664-788: query i attends
// cache rows [first_i, past_len + i]; head_dim 64, 96 — staged as 128 — and 128; linear and ring
// planes), different shape of the pipeline:
//   * Work item = (pair of query tiles A and B = 2 x QT consecutive queries, KV head, key split).
//     Both tiles are contracted against the SAME staged K and V tiles, so shared-memory and L2
//     traffic per flop halve.
//   * Softmax group A (warps 0-3) owns the rows of tile A, group B (warps 4-7) those of tile B:
//     one thread per row, all 128 score columns — no exchange between threads. The two groups
//     are a tile-phase apart by construction: while A runs exp2 on its scores the tensor core
//     runs  O_B += P_B·V  and  S_B = Q_B·K^T  for the other tile, and vice versa, so neither the
//     tensor pipe nor the MUFU pipe waits for the other's latency chain.
//   * Tensor memory (512 columns): S_A [0,128)  S_B [128,256)  O_A [256,384)  O_B [384,512).
//     P (packed fp16, 64 columns) is written over the first half of its own S: the score MMA of
//     the next tile is issued after P·V of this one on the same in-order pipe, so S is dead by
//     the time P lands, and P is dead by the time the next S lands.
//   * Issue order of warp 9 per key tile j:  PV_A(j) QK_A(j+1)  PV_B(j) QK_B(j+1). The issuing
//     thread (like the TMA producer's) is picked with elect.sync, which lets the compiler keep the
//     operand descriptors in uniform registers: a batch of 16 MMAs then issues in ~740 cycles and
//     runs asynchronously, against 1 340 cycles of issue when the thread was picked by lane id.
//   * exp2 is the narrow pipe (16 per clock per SM, as many cycles per tile as both MMAs): 3 of
//     every 8 element pairs take a degree-3 polynomial on the FMA pipe instead (ex2_emu2).
//   * O accumulates in tensor memory for the whole item; a row is rescaled in place (by its own
//     thread) only when its maximum outgrows the reference by more than 2^8.
//   * All waits are bounded mbarrier waits reporting through the status word; tensor memory is
//     freed on every path.
#pragma once

#include "hkv_prefill_tc.cuh"

namespace hkv {

constexpr int kPf2KStages = 2;
constexpr int kPf2VStages = 2;
// 12 warps: 0-3 softmax group A, 4-7 group B, 8 TMA producer, 9 MMA issuer, 10-11 only complete the
// third warpgroup so that it can hand its registers to the softmax warps (setmaxnreg works on whole
// warpgroups): 168 registers per thread at launch, 192 for the softmax rows, 120 for the rest.
constexpr int kPf2Threads = 384;
#ifndef HKV_PF2_EMU
#define HKV_PF2_EMU 3
#endif
constexpr int kPf2EmuOf8 = HKV_PF2_EMU;   // pairs of every 8 whose exp2 runs on the FMA pipe


constexpr int kPf2MaxPairs = 1024;   // tile pairs of a chunk the equal-span schedule can tabulate (36 864 queries at group 7)

__host__ __device__ constexpr size_t prefill_tc2_smem_bytes(int HD) {
    return 1024 + (size_t)(2 + kPf2KStages + kPf2VStages) * kPfRows * HD * 2 + 32 * 8 + 16 + 4 * 8 * 4 + (kPf2MaxPairs + 1) * 4 + 16;
}

// CTA that owns work unit x when W units are cut into `grid` equal contiguous spans with
// boundaries floor(W * c / grid): the largest c whose boundary is <= x.
__host__ __device__ inline int prefill_span_owner(long long x, long long W, int grid) {
    return (int)(((x + 1) * grid + W - 1) / W - 1);
}

// tcgen05.wait::ld that also names the registers of the load it completes, so that no use of
// them can be scheduled above the wait.
__device__ __forceinline__ void tc_wait_ld_dep(uint32_t (&v)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                   "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
                   "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
                   "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
                 :
                 : "memory");
}

// 2^x for two values on the FMA pipe (the MUFU pipe is the narrowest unit of the softmax: 16
// ex2 per clock per SM). x is clamped to [-100, +inf); callers keep x <= ~9. Round-to-nearest
// split x = n + f, f in [-0.5, 0.5], by adding 1.5*2^23; 2^f by a degree-3 minimax polynomial
// (max relative error 7.5e-5, below half an ulp of the fp16 the result is rounded to); 2^n by
// adding n to the exponent field.
__device__ __forceinline__ void ex2_emu2(float& p0, float& p1, float x0, float x1) {
    x0 = fmaxf(x0, -100.0f);
    x1 = fmaxf(x1, -100.0f);
    uint32_t t0, t1, q0, q1;
    asm("{\n\t.reg .b64 rx, rt, rr, rf, rp, rc;\n\t"
        "mov.b64 rx, {%4, %5};\n\t"
        "mov.b64 rc, {0f4B400000, 0f4B400000};\n\t"      // 12582912.0
        "add.rn.f32x2 rt, rx, rc;\n\t"                    // n in the low mantissa bits
        "sub.rn.f32x2 rr, rt, rc;\n\t"                    // n as a float
        "sub.rn.f32x2 rf, rx, rr;\n\t"                    // f = x - n
        "mov.b64 rp, {0f3D61FB59, 0f3D61FB59};\n\t"      // 0.055171344
        "mov.b64 rc, {0f3E786ED8, 0f3E786ED8};\n\t"      // 0.24261034
        "fma.rn.f32x2 rp, rp, rf, rc;\n\t"
        "mov.b64 rc, {0f3F31798D, 0f3F31798D};\n\t"      // 0.69326097
        "fma.rn.f32x2 rp, rp, rf, rc;\n\t"
        "mov.b64 rc, {0f3F7FFB4A, 0f3F7FFB4A};\n\t"      // 0.9999281
        "fma.rn.f32x2 rp, rp, rf, rc;\n\t"
        "mov.b64 {%0, %1}, rt;\n\t"
        "mov.b64 {%2, %3}, rp;\n\t}"
        : "=r"(t0), "=r"(t1), "=r"(q0), "=r"(q1)
        : "f"(x0), "f"(x1));
    p0 = __uint_as_float(q0 + (t0 << 23));
    p1 = __uint_as_float(q1 + (t1 << 23));
}

// MMA wrappers for the issuing thread's inner loops: the accumulate flag is an immediate and the
// 64-bit shared-memory descriptors are passed as (low, high) words — every descriptor of this kernel
// has the same high word (8-row group stride 1024 B, version, 128-byte swizzle), and the low word
// (start address, leading-dimension offset) moves by a compile-time constant per instruction, so
// the loop costs one 32-bit add per operand instead of 64-bit descriptor arithmetic.
template <bool ACC>
__device__ __forceinline__ void tc_mma_ss_i(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(ACC ? 1 : 0)
        : "memory");
}
template <bool ACC>
__device__ __forceinline__ void tc_mma_ts_i(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(ACC ? 1 : 0)
        : "memory");
}

template <int HD>
__global__ void __launch_bounds__(kPf2Threads, 1)
hkv_prefill_tc2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const PrefillTcArgs a) {
    static_assert(HD == 64 || HD == 128, "head_dim 64 or 128");
    constexpr int NCH = HD / 64;                       // 64-half column blocks
    constexpr int CHUNK_BYTES = kPfRows * 128;         // one column block of a 128-row tile
    constexpr int TILE_BYTES = kPfRows * HD * 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t COL_S = 0, COL_O = 256;         // + 128 * group
    constexpr uint32_t IDESC_QK = (1u << 4) | ((uint32_t)(kPfKeys >> 3) << 17) | ((uint32_t)(kPfRows >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(kPfRows >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_gen = smem;                                    // Q tiles A, B
    uint8_t* k_gen = smem + 2 * TILE_BYTES;                   // kPf2KStages K tiles
    uint8_t* v_gen = k_gen + kPf2KStages * TILE_BYTES;        // kPf2VStages V tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_gen + kPf2VStages * TILE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
    const uint32_t q_smem = smem_u32(q_gen), k_smem = smem_u32(k_gen), v_smem = smem_u32(v_gen);
    const uint32_t bar0 = smem_u32(bars);
    // barrier map (8 bytes each)
    const uint32_t B_QFULL = bar0, B_QEMPTY = bar0 + 8;
    const uint32_t B_KFULL = bar0 + 16;     // [2]
    const uint32_t B_KEMPTY = bar0 + 32;    // [2]
    const uint32_t B_VFULL = bar0 + 48;     // [2]
    const uint32_t B_VEMPTY = bar0 + 64;    // [2]
    const uint32_t B_SFULL = bar0 + 80;     // [group]
    const uint32_t B_PFULL = bar0 + 96;     // [group]
    const uint32_t B_OFULL = bar0 + 112;    // [group] last P·V of an item has completed
    const uint32_t B_DONE = bar0 + 128;
    // Work queue: the producer decides what the CTA works on and hands each piece of work to the
    // other roles through four shared-memory slots as a descriptor
    //   {pair of query tiles, kv head, first key tile, key tiles, part index, parts of the item}.
    // Two schedules: (a) whole items (or equal key-range splits of them) taken off a global counter,
    // longest first — whichever CTA is free takes the next; (b) whole items for as many full rounds of
    // the grid as there are, then equal spans for the rest: the key tiles of the remaining items form
    // one line, cut into equal contiguous spans, one per CTA, so the last round costs every CTA the same
    // number of tile steps instead of leaving most SMs idle; an item that straddles a cut is finished by
    // two (or more) CTAs, each writing a partial row that the merge kernel combines.
    const uint32_t B_QF = bar0 + 144;       // [4] slot holds a descriptor (first word -1 = no more work)
    const uint32_t B_QE = bar0 + 176;       // [4] slot read by the MMA issuer and the 8 softmax warps
    volatile int* q_items = reinterpret_cast<volatile int*>(tmem_slot + 4);   // [4][8]
    int* pre = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 4 + 32));   // [n_qtiles + 1] (equal spans)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(B_QFULL, 1); mbar_init(B_QEMPTY, 1);
        for (int s = 0; s < kPf2KStages; ++s) { mbar_init(B_KFULL + 8 * s, 1); mbar_init(B_KEMPTY + 8 * s, 1); }
        for (int s = 0; s < kPf2VStages; ++s) { mbar_init(B_VFULL + 8 * s, 1); mbar_init(B_VEMPTY + 8 * s, 1); }
        for (int g = 0; g < 2; ++g) { mbar_init(B_SFULL + 8 * g, 1); mbar_init(B_PFULL + 8 * g, 128); mbar_init(B_OFULL + 8 * g, 1); }
        mbar_init(B_DONE, 1);
        for (int i = 0; i < 4; ++i) { mbar_init(B_QF + 8 * i, 1); mbar_init(B_QE + 8 * i, 9); }
        fence_mbar_init();
        tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
    }
    if (warp == 9) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // a.QT = queries per 128-row tile; a.n_qtiles counts PAIRS of tiles here
    const int QT2 = 2 * a.QT;
    const int n_items = a.n_qtiles * a.KVH * a.splits;
    const int kv_valid = prefill_kv_valid(a);

    // Key-tile range of a tile pair and split (identical in every role); tiles count logical positions.
    auto tile_span = [&](int qt, int sp, int& kt_lo, int& nt) { prefill_tile_span(a, QT2, kPfKeys, qt, sp, kt_lo, nt); };
    auto decode_item = [&](int item, int& qt, int& kvh, int& sp) {
        sp = item % a.splits;
        const int rest = item / a.splits;
        qt = a.n_qtiles - 1 - rest / a.KVH;   // longest spans first
        kvh = rest % a.KVH;
    };

    // Consumers of the queue: entry k lives in slot k % 4, phase k / 4.
    auto queue_wait = [&](uint32_t k) -> bool { return mbar_wait(B_QF + 8 * (k & 3), (k >> 2) & 1, a.status); };

    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 120;");
    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        const int n_pairs = a.n_qtiles;
        if (a.streamk) {
            // pre[j] = key tiles of the pairs before j in processing order (pair n-1-j: longest first)
            int carry = 0;
            for (int j0 = 0; j0 < n_pairs; j0 += 32) {
                const int j = j0 + lane;
                int kt0, v = 0;
                if (j < n_pairs) prefill_item_tiles(a, QT2, kPfKeys, n_pairs - 1 - j, kt0, v);
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int u = __shfl_up_sync(0xffffffffu, v, o);
                    if (lane >= o) v += u;
                }
                if (j < n_pairs) pre[j + 1] = carry + v;
                carry += __shfl_sync(0xffffffffu, v, 31);
            }
            if (lane == 0) pre[0] = 0;
            __syncwarp();
        }
        if (elect_one()) {
            uint32_t gt = 0, it = 0, q_it = 0, qk = 0;
            bool ok = true, q_pending = false;
            auto publish = [&](int qt, int kvh, int kt_lo, int nt, int part, int nparts) -> bool {
                const uint32_t slot = qk & 3;
                if (qk >= 4 && !mbar_wait(B_QE + 8 * slot, ((qk >> 2) - 1) & 1, a.status)) return false;
                volatile int* d = q_items + slot * 8;
                d[0] = qt; d[1] = kvh; d[2] = kt_lo; d[3] = nt; d[4] = part; d[5] = nparts;
                mbar_arrive(B_QF + 8 * slot);
                ++qk;
                return true;
            };
            // One piece of work: announce it, load its two query tiles, stream its K/V tiles.
            auto run_piece = [&](int qt, int kvh, int kt_lo, int nt, int part, int nparts) {
                if (!publish(qt, kvh, kt_lo, nt, part, nparts)) { ok = false; return; }
                if (!mbar_wait(B_QEMPTY, (it & 1) ^ 1, a.status)) { ok = false; return; }
                mbar_expect_tx(B_QFULL, (uint32_t)(2 * NCH * a.QT * a.G * 128));
#pragma unroll
                for (int t2 = 0; t2 < 2; ++t2)
#pragma unroll
                    for (int c = 0; c < NCH; ++c)
                        tma_load_3d(q_smem + t2 * TILE_BYTES + c * CHUNK_BYTES, &tm_q, B_QFULL, c * 64, kvh * a.G,
                                    qt * QT2 + t2 * a.QT);
                q_pending = true;
                q_it = it;
                for (int t = 0; t < nt; ++t, ++gt) {
                    const int row = prefill_tile_row(a, (kt_lo + t) * kPfKeys);
                    const uint32_t ks = gt % kPf2KStages, ku = gt / kPf2KStages;
                    if (!mbar_wait(B_KEMPTY + 8 * ks, (ku & 1) ^ 1, a.status)) { ok = false; return; }
                    mbar_expect_tx(B_KFULL + 8 * ks, TILE_BYTES);
#pragma unroll
                    for (int c = 0; c < NCH; ++c)
                        tma_load_4d(k_smem + ks * TILE_BYTES + c * CHUNK_BYTES, &tm_k, B_KFULL + 8 * ks, c * 64, kvh,
                                    row, 0);
                    const uint32_t vs = gt % kPf2VStages, vu = gt / kPf2VStages;
                    if (!mbar_wait(B_VEMPTY + 8 * vs, (vu & 1) ^ 1, a.status)) {
                        mbar_wait(B_KFULL + 8 * ks, ku & 1, a.status);   // the K copy above is in flight
                        ok = false;
                        return;
                    }
                    mbar_expect_tx(B_VFULL + 8 * vs, TILE_BYTES);
#pragma unroll
                    for (int c = 0; c < NCH; ++c)
                        tma_load_4d(v_smem + vs * TILE_BYTES + c * CHUNK_BYTES, &tm_v, B_VFULL + 8 * vs, c * 64, kvh,
                                    row, 0);
                }
                ++it;
            };
            if (a.streamk) {
                // Phase 1: the first sk_whole items (the longest, a whole number of rounds of the grid) run
                // whole, taken off the shared counter: CTAs sweep the keys in rough lockstep, which keeps the
                // K/V tiles that many items share in L2. Item I = (pair j = I / KVH, kv head I % KVH).
                for (int item = blockIdx.x; item < a.sk_whole && ok; item = (int)gridDim.x + atomicAdd(a.item_counter, 1)) {
                    const int j = item / a.KVH;
                    int kt0, T;
                    prefill_item_tiles(a, QT2, kPfKeys, n_pairs - 1 - j, kt0, T);
                    run_piece(n_pairs - 1 - j, item % a.KVH, kt0, T, 0, 1);
                }
                // Phase 2: the remaining items (fewer than one round) form one line of key tiles that is cut
                // into sk_grid equal spans; this CTA takes span [u0, u1). Item (j, kvh) starts at
                // KVH * pre[j] + kvh * T(j); units are counted from the first item of the tail.
                const int j0 = a.sk_whole / a.KVH, kvh0 = a.sk_whole % a.KVH;
                const long long line0 = j0 < n_pairs ? (long long)a.KVH * pre[j0] + (long long)kvh0 * (pre[j0 + 1] - pre[j0]) : 0;
                const long long W = (long long)pre[n_pairs] * a.KVH - line0;
                const int sg = a.sk_grid;
                if (ok && j0 < n_pairs && (int)blockIdx.x < sg && W > 0) {
                    const long long u0 = line0 + W * blockIdx.x / sg, u1 = line0 + W * (blockIdx.x + 1) / sg;
                    if (u0 < u1) {
                        int lo = j0, hi = n_pairs - 1;
                        while (lo < hi) {
                            const int mid = (lo + hi + 1) >> 1;
                            if ((long long)a.KVH * pre[mid] <= u0) lo = mid; else hi = mid - 1;
                        }
                        int j = lo, T = pre[j + 1] - pre[j];
                        const long long rem = u0 - (long long)a.KVH * pre[j];
                        int kvh = (int)(rem / T), off = (int)(rem % T);
                        for (long long u = u0; u < u1 && ok;) {
                            const long long left = u1 - u;
                            const int nt = (long long)(T - off) < left ? T - off : (int)left;
                            const long long P = (long long)a.KVH * pre[j] + (long long)kvh * T - line0;
                            const int c_first = prefill_span_owner(P, W, sg);
                            const int c_last = prefill_span_owner(P + T - 1, W, sg);
                            int kt0, tdummy;
                            prefill_item_tiles(a, QT2, kPfKeys, n_pairs - 1 - j, kt0, tdummy);
                            run_piece(n_pairs - 1 - j, kvh, kt0 + off, nt, (int)blockIdx.x - c_first, c_last - c_first + 1);
                            u += nt;
                            off = 0;
                            if (++kvh == a.KVH) {
                                kvh = 0;
                                if (++j < n_pairs) T = pre[j + 1] - pre[j];
                            }
                        }
                    }
                }
            } else {
                // first item = this CTA's index, then whatever the shared counter hands out
                for (int item = blockIdx.x; item < n_items && ok; item = (int)gridDim.x + atomicAdd(a.item_counter, 1)) {
                    int qt, kvh, sp, kt_lo, nt;
                    decode_item(item, qt, kvh, sp);
                    tile_span(qt, sp, kt_lo, nt);
                    if (a.out_parts > 0) run_piece(qt, kvh, kt_lo, nt, a.out_part * a.splits + sp, a.out_parts * a.splits);
                    else run_piece(qt, kvh, kt_lo, nt, sp, a.splits);
                }
            }
            publish(-1, 0, 0, 0, 0, 0);   // no more work (also after a wait that ran out: the other roles leave at once)
            // drain this thread's outstanding copies before the CTA retires (tiles 0..gt-1 were issued)
            if (q_pending) mbar_wait(B_QFULL, q_it & 1, a.status);
            for (uint32_t i = 1; i <= (uint32_t)kPf2KStages && i <= gt; ++i) {
                const uint32_t g = gt - i;
                mbar_wait(B_KFULL + 8 * (g % kPf2KStages), (g / kPf2KStages) & 1, a.status);
            }
            for (uint32_t i = 1; i <= (uint32_t)kPf2VStages && i <= gt; ++i) {
                const uint32_t g = gt - i;
                mbar_wait(B_VFULL + 8 * (g % kPf2VStages), (g / kPf2VStages) & 1, a.status);
            }
        }
    } else if (warp == 9) {
        // ------------------------------ MMA issuer ------------------------------
        if (elect_one()) {
            uint32_t gt = 0, it = 0;
            bool ok = true;
            const uint64_t qdesc0 = umma_desc_sw128(q_smem, 16), kdesc0 = umma_desc_sw128(k_smem, 16);
            const uint64_t vdesc0 = umma_desc_sw128(v_smem, CHUNK_BYTES);
            const uint32_t desc_hi = (uint32_t)(qdesc0 >> 32);
            const uint32_t q_lo = (uint32_t)qdesc0, k_lo = (uint32_t)kdesc0, v_lo = (uint32_t)vdesc0;
            const int ksteps = (a.HD + 15) / 16;   // k-steps holding real dimensions (zero-filled ones are skipped)
            // S_grp = Q_grp · K(g)^T   (the K tile must have been waited for)
            auto issue_qk = [&](uint32_t g, int grp) {
                const uint32_t kd = k_lo + (((g % kPf2KStages) * TILE_BYTES) >> 4);
                const uint32_t qd = q_lo + ((grp * TILE_BYTES) >> 4);
                const uint32_t d = tmem + COL_S + 128u * grp;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t off = (uint32_t)(((kk / 4) * CHUNK_BYTES + (kk % 4) * 32) >> 4);
                    if (kk == 0) tc_mma_ss_i<false>(d, qd + off, kd + off, desc_hi, IDESC_QK);
                    else if (kk < ksteps) tc_mma_ss_i<true>(d, qd + off, kd + off, desc_hi, IDESC_QK);
                }
                tc_commit(B_SFULL + 8 * grp);
            };
            // O_grp (+)= P_grp · V(g)   (P lives in the first 64 columns of S_grp)
            auto issue_pv = [&](uint32_t g, int grp, bool accumulate) {
                const uint32_t vd = v_lo + (((g % kPf2VStages) * TILE_BYTES) >> 4);
                const uint32_t pbase = tmem + COL_S + 128u * grp, d = tmem + COL_O + 128u * grp;
                if (accumulate) tc_mma_ts_i<true>(d, pbase, vd, desc_hi, IDESC_PV);
                else tc_mma_ts_i<false>(d, pbase, vd, desc_hi, IDESC_PV);
#pragma unroll
                for (int kk = 1; kk < kPfKeys / 16; ++kk)
                    tc_mma_ts_i<true>(d, pbase + kk * 8, vd + (uint32_t)((kk * 2048) >> 4), desc_hi, IDESC_PV);
            };
            for (; ok; ++it) {
                if (!queue_wait(it)) { ok = false; break; }
                const int qt = q_items[(it & 3) * 8], nt = q_items[(it & 3) * 8 + 3];
                mbar_arrive(B_QE + 8 * (it & 3));
                if (qt < 0) break;
                if (!mbar_wait(B_QFULL, it & 1, a.status) ||
                    !mbar_wait(B_KFULL + 8 * (gt % kPf2KStages), (gt / kPf2KStages) & 1, a.status)) { ok = false; break; }
                tc_fence_after();
                issue_qk(gt, 0);
                issue_qk(gt, 1);
                tc_commit(B_KEMPTY + 8 * (gt % kPf2KStages));
                if (nt == 1) tc_commit(B_QEMPTY);
                for (int t = 0; t < nt && ok; ++t, ++gt) {
                    const bool more = t + 1 < nt;
                    const uint32_t vs = gt % kPf2VStages, ks1 = (gt + 1) % kPf2KStages;
                    // the operand tiles of this step first (they land long before P does), so that
                    // nothing stands between the arrival of P and the first MMA
                    if (!mbar_wait(B_VFULL + 8 * vs, (gt / kPf2VStages) & 1, a.status) ||
                        (more && !mbar_wait(B_KFULL + 8 * ks1, ((gt + 1) / kPf2KStages) & 1, a.status))) { ok = false; break; }
#pragma unroll
                    for (int grp = 0; grp < 2; ++grp) {
                        if (!mbar_wait(B_PFULL + 8 * grp, gt & 1, a.status)) { ok = false; break; }
                        tc_fence_after();
                        issue_pv(gt, grp, t > 0);
                        if (!more) tc_commit(B_OFULL + 8 * grp);        // the item's output of this tile is complete
                        if (grp == 1) tc_commit(B_VEMPTY + 8 * vs);     // both tiles have consumed V(g)
                        if (more) {
                            issue_qk(gt + 1, grp);
                            if (grp == 1) {
                                tc_commit(B_KEMPTY + 8 * ks1);
                                if (t + 2 == nt) tc_commit(B_QEMPTY);   // last score MMAs of the item issued
                            }
                        }
                    }
                }
            }
            // every MMA issued above has completed before tensor memory is freed
            tc_commit(B_DONE);
            mbar_wait(B_DONE, 0, a.status);
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");
        // ------------------------------ softmax / output rows ------------------------------
        const int quad = warp & 3, grp = warp >> 2;
        const int r = quad * 32 + lane;            // row of the tile = lane of tensor memory
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const uint32_t s_addr = tmem + lane_sel + COL_S + 128u * grp;
        const uint32_t o_addr = tmem + lane_sel + COL_O + 128u * grp;
        const uint32_t b_sfull = B_SFULL + 8 * grp, b_pfull = B_PFULL + 8 * grp, b_ofull = B_OFULL + 8 * grp;
        const int ql = r / a.G, g = r % a.G;
        uint32_t gt = 0, si = 0;   // tiles seen, items done (barrier phases)
        bool ok = true;            // kept warp-uniform: a wait that ran out for any lane stops the warp
        for (uint32_t qk = 0; ok; ++qk) {
            ok = __all_sync(0xffffffffu, queue_wait(qk));
            if (!ok) break;
            const volatile int* dsc = q_items + (qk & 3) * 8;
            const int qt = dsc[0], kvh = dsc[1], kt_lo = dsc[2], nt = dsc[3], part = dsc[4], nparts = dsc[5];
            __syncwarp();
            if (lane == 0) mbar_arrive(B_QE + 8 * (qk & 3));
            if (qt < 0) break;
            const int qi = qt * QT2 + grp * a.QT + ql;
            const bool row_valid = ql < a.QT && qi < a.S_new;
            const int qpos = a.past_len + qi;
            const int first_row = a.window > 0 ? (qpos + 1 - a.window > 0 ? qpos + 1 - a.window : 0) : 0;
            const int qlim = prefill_last_key(a, qpos);  // never attend rows past a linear plane
            // m_ref: the reference maximum P and O are scaled by; it moves (and O is rescaled) only
            // when a tile's maximum exceeds it by more than 2^8 — fp16 holds P up to that factor.
            float m_ref = kNegBig, l_run = 0.0f;

            for (int t = 0; t < nt; ++t, ++gt) {
                ok = __all_sync(0xffffffffu, ok && mbar_wait(b_sfull, gt & 1, a.status));
                if (!ok) continue;
                tc_fence_after();
                // ---- the row's 128 scores, read once (mask bounds are computed under the loads) ----
                uint32_t sv[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(sv[c], s_addr + c * 32);
                const int kstart = (kt_lo + t) * kPfKeys;
                const int lo = first_row - kstart, hi = qlim - kstart;   // attended columns [lo, hi]
                const bool all_in = __all_sync(0xffffffffu, lo <= 0 && hi >= kPfKeys - 1);
#pragma unroll
                for (int c = 0; c < 4; ++c) tc_wait_ld_dep(sv[c]);
                // ---- row maximum of the raw scores (the scale is positive) ----
                float mx;
                {
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;   // independent chains
                    if (all_in) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                m0 = fmax3(m0, __uint_as_float(sv[c][j]), __uint_as_float(sv[c][j + 1]));
                                m1 = fmax3(m1, __uint_as_float(sv[c][j + 2]), __uint_as_float(sv[c][j + 3]));
                                m2 = fmax3(m2, __uint_as_float(sv[c][j + 4]), __uint_as_float(sv[c][j + 5]));
                                m3 = fmax3(m3, __uint_as_float(sv[c][j + 6]), __uint_as_float(sv[c][j + 7]));
                            }
                    } else {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const int col = c * 32 + j;
                                const float sc = (col >= lo && col <= hi) ? __uint_as_float(sv[c][j]) : -INFINITY;
                                sv[c][j] = __float_as_uint(sc);
                                m0 = fmaxf(m0, sc);
                            }
                    }
                    mx = fmaxf(fmax3(m0, m1, m2), m3);
                }
                mx *= a.scale_log2;
                const bool move = mx > m_ref + 8.0f;
                if (__any_sync(0xffffffffu, move)) {
                    const float m_to = move ? mx : m_ref;
                    const float alpha = ex2_approx(m_ref - m_to);   // 1 for rows that keep their reference
                    // The score MMA of this tile was issued after P·V of the previous one, so O is
                    // complete up to tile t-1 here.
                    if (t > 0) tmem_scale_columns(o_addr, HD / 32, alpha);
                    l_run *= alpha;
                    m_ref = m_to;
                }
                // ---- p = 2^(s*scale - m_ref), row sum, P back to tensor memory as packed fp16 ----
                float lsum0 = 0.0f, lsum1 = 0.0f, lsum2 = 0.0f, lsum3 = 0.0f;
                const float neg_m = -m_ref;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        float x0, x1, x2, x3;
                        ffma2_bcast(x0, x1, __uint_as_float(sv[c][j]), __uint_as_float(sv[c][j + 1]), a.scale_log2, neg_m);
                        ffma2_bcast(x2, x3, __uint_as_float(sv[c][j + 2]), __uint_as_float(sv[c][j + 3]), a.scale_log2, neg_m);
                        float p0, p1, p2, p3;
                        if (((j / 4) * 2) % 8 < kPf2EmuOf8) ex2_emu2(p0, p1, x0, x1);
                        else { p0 = ex2_approx(x0); p1 = ex2_approx(x1); }
                        if (((j / 4) * 2 + 1) % 8 < kPf2EmuOf8) ex2_emu2(p2, p3, x2, x3);
                        else { p2 = ex2_approx(x2); p3 = ex2_approx(x3); }
                        fadd2_acc(lsum0, lsum1, p0, p1);
                        fadd2_acc(lsum2, lsum3, p2, p3);
                        pk[j / 2] = pack_half2(p0, p1);
                        pk[j / 2 + 1] = pack_half2(p2, p3);
                    }
                    // P columns [16c, 16c+16) of this row overwrite its scores, all of which are in registers
                    tmem_st16(s_addr + c * 16, pk);
                }
                tc_wait_st();
                l_run += (lsum0 + lsum1) + (lsum2 + lsum3);
                // cache rows of this tile past the last written position may hold stale bits: group A
                // zeroes them in the staged V tile (before its arrival below, which precedes both
                // output MMAs of the tile) so that 0 * garbage cannot produce NaN
                const int tile0 = (kt_lo + t) * kPfKeys;
                if (grp == 0 && tile0 + kPfKeys > kv_valid) {
                    const uint32_t vs = gt % kPf2VStages;
                    ok = __all_sync(0xffffffffu, mbar_wait(B_VFULL + 8 * vs, (gt / kPf2VStages) & 1, a.status));
                    if (!ok) continue;
                    uint8_t* vt = v_gen + (size_t)vs * TILE_BYTES;
                    const int first_bad = kv_valid > tile0 ? kv_valid - tile0 : 0;
                    for (int idx = first_bad * 8 * NCH + tid; idx < kPfKeys * 8 * NCH; idx += 128) {
                        const int row = idx / (8 * NCH), u = idx % (8 * NCH);
                        *reinterpret_cast<uint4*>(vt + (u / 8) * CHUNK_BYTES + row * 128 + (u % 8) * 16) =
                            make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                tc_fence_before();
                mbar_arrive(b_pfull);
            }
            // Wait for the item's last P·V of this tile, then write the row out.
            ok = __all_sync(0xffffffffu, ok && mbar_wait(b_ofull, si & 1, a.status));
            ++si;
            if (!ok) continue;
            tc_fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            float* prow = nullptr;
            __half* op = nullptr;
            if (row_valid) {
                if (nparts > 1) prow = a.part + (((long long)qi * a.part_stride + part) * a.H + (long long)kvh * a.G + g) * (a.HD + 2);
                else op = a.out + ((long long)qi * a.H + (long long)kvh * a.G + g) * a.HD;
                // how many partial rows the merge kernel finds for this (query, kv head)
                if (a.row_parts && part == 0 && g == 0) a.row_parts[(long long)qi * a.KVH + kvh] = nparts;
            }
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(v, o_addr + c * 32);
                tc_wait_ld_dep(v);
                if (c * 32 >= a.HD) continue;          // zero-filled padding columns (head_dim 96)
                if (prow) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2)
                        *reinterpret_cast<float2*>(prow + c * 32 + j) = make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                } else if (op) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 w;
                        w.x = pack_half2(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
                        w.y = pack_half2(__uint_as_float(v[j + 2]) * inv, __uint_as_float(v[j + 3]) * inv);
                        w.z = pack_half2(__uint_as_float(v[j + 4]) * inv, __uint_as_float(v[j + 5]) * inv);
                        w.w = pack_half2(__uint_as_float(v[j + 6]) * inv, __uint_as_float(v[j + 7]) * inv);
                        *reinterpret_cast<uint4*>(op + c * 32 + j) = w;
                    }
                }
            }
            if (prow) {
                prow[a.HD] = m_ref;
                prow[a.HD + 1] = l_run;
            }
            tc_fence_before();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace hkv
