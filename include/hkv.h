/* hkv.h — C ABI of libhkv: KV-cache append + cached grouped-query attention for
 * NVIDIA B200 (sm_100a), a drop-in for that one hot path of the Héctor / HELIOS engine.
 *
 * Conventions
 *   - Every entry point returns an hkv_status (0 = ok); nothing throws, nothing is
 *     printed. hkv_ctx_last_error() gives the text of the last failure of a context.
 *   - All tensors are IEEE binary16 ("fp16") in device memory, passed as void*;
 *     positions are int32 in DEVICE memory (one per sequence); `stream` is a
 *     cudaStream_t passed as void* (NULL = the legacy default stream).
 *   - Launch entry points only enqueue work on `stream`: no allocation, no
 *     synchronisation, no host read of device memory. They may be called while the
 *     stream is being captured into a CUDA graph; per-step variation then comes only
 *     from the device-side position arrays. hkv_ctx_create / destroy / *_host /
 *     hkv_ctx_device_status are NOT capturable (they allocate or synchronise).
 *   - There is no CPU path. Without a usable CUDA device every call fails with
 *     HKV_ERR_NO_DEVICE or HKV_ERR_CUDA.
 *
 * Layouts (row-major, matching the reference engine; paths below are relative to the
 * reference project root)
 *   q, out        [batch, 1, num_heads, head_dim]           kernels/attention.cu:156-159
 *   k/v plane     [batch, slots, num_kv_heads, head_dim]    src/kv_cache.hpp:175-189
 *   k_new, v_new  [batch, seq_new, num_kv_heads, head_dim]  kernels/attention.cu:1092-1094
 *   prefill q/out [seq_new, num_heads, head_dim], batch 1   kernels/attention.cu:665-668
 */
#ifndef HKV_H_
#define HKV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HKV_ABI_VERSION 2

typedef enum hkv_status {
    HKV_OK = 0,
    HKV_ERR_INVALID_ARG = 1, /* null pointer, negative size, unknown enum value          */
    HKV_ERR_GEOMETRY = 2,    /* head geometry the reference op would also reject, or a
                                combination this library does not implement              */
    HKV_ERR_ALIGNMENT = 3,   /* a pointer or stride is not a multiple of 2 bytes         */
    HKV_ERR_CUDA = 4,        /* a CUDA runtime / driver call failed                      */
    HKV_ERR_NO_DEVICE = 5,   /* no CUDA device, or not compute capability 10.x           */
    HKV_ERR_WORKSPACE = 6,   /* caller-supplied workspace too small                      */
    HKV_ERR_TOO_LARGE = 7,   /* a size exceeds a documented maximum                      */
    HKV_ERR_DEVICE_FAULT = 8 /* the device status word reports a bounded wait that ran out */
} hkv_status;

typedef enum hkv_layout {
    HKV_LAYOUT_LINEAR = 0, /* row = position; rows >= slots are dropped on append
                              (kernels/attention.cu:1143-1144)                           */
    HKV_LAYOUT_RING = 1    /* row = position mod slots (sliding-window layers). Not in the
                              reference; results equal the reference's linear cache with
                              window_size = slots                                        */
} hkv_layout;

typedef enum hkv_kernel_select {
    HKV_KERNEL_AUTO = 0,    /* TMA-staged tensor-tile kernel when the geometry allows    */
    HKV_KERNEL_GENERIC = 1, /* force the any-geometry SIMT kernel                        */
    HKV_KERNEL_TMA = 2      /* require the TMA kernel; HKV_ERR_GEOMETRY if not eligible  */
} hkv_kernel_select;

/* Geometry of one attention layer's cache and op. Zero-initialise, then fill in. */
typedef struct hkv_geometry {
    int32_t batch;        /* sequences per call (the reference op is always 1,
                             kernels/register_kernels.cpp:870)                           */
    int32_t num_heads;    /* query heads H                                               */
    int32_t num_kv_heads; /* KV heads; H % KVH == 0 (kernels/register_kernels.cpp:858)   */
    int32_t head_dim;     /* 1..512 (kernels/register_kernels.cpp:858)                   */
    int32_t slots;        /* rows per sequence in a plane = the reference's max_seq_len  */
    int32_t window_size;  /* 0 = attend everything; W = last W positions
                             (kernels/attention.cu:385)                                  */
    int32_t layout;       /* hkv_layout                                                  */
    int32_t chunk_tiles;  /* split-K work item size in 64-row tiles; 0 = auto            */
    int64_t batch_stride_elems; /* elements between sequences in a plane; 0 = dense      */
    /* Sequence-split sharding of ONE logical cache over several GPUs: logical blocks of
     * `shard_block` positions are dealt round-robin, block j lives on rank j % shard_count
     * as local block j / shard_count. shard_count <= 1 means not sharded.               */
    int32_t shard_rank;
    int32_t shard_count;
    int32_t shard_block;  /* multiple of 64                                              */
    int32_t kernel_select; /* hkv_kernel_select                                          */
    int32_t max_seq_new;  /* largest seq_new hkv_prefill_attention may split by key range
                             (allocates seq_new*4*H*(HD+2)*4 bytes of partials); 0 = no split */
    int32_t flags;        /* HKV_FLAG_* bits                                             */
    /* Overrides of choices the library otherwise makes itself (parity tests run every
     * variant through them); 0 = automatic.                                             */
    int32_t tune_prefill_splits; /* key-range splits of a prefill work item, 1..4; clamped to
                                    what the plan allows                                 */
    int32_t tune_prefill_kernel; /* 1 = one query tile in flight per CTA, 2 = two        */
    int32_t tune_tma_groups;     /* shape of the TMA decode kernel: 1 = two CTAs per SM with one
                                    consumer group each, 2 = one CTA with two groups, 3 = one CTA
                                    with one group and the whole shared memory as its ring */
    /* Decode-side calls (one new token per sequence) may read q and k_new / v_new straight out of a
     * fused QKV activation [batch][num_heads*head_dim | num_kv_heads*head_dim | num_kv_heads*head_dim]
     * — the zero-copy split the reference does for batch 1 only (kernels/register_kernels.cpp:587-593):
     * elements between consecutive sequences' q rows, and between their k_new (= v_new) rows.
     * 0 = dense ([batch, num_heads, head_dim] and [batch, num_kv_heads, head_dim]). The outputs stay
     * dense. Calls with several new tokens per sequence (hkv_append with seq_new > 1, prefill, rope)
     * take dense tensors. */
    int32_t q_seq_stride_elems;
    int32_t new_kv_seq_stride_elems;
    int32_t reserved[1];
} hkv_geometry;

/* hkv_geometry.flags */
/* The device position arrays hold ONE int32 that every sequence of the batch reads, as the
 * reference's kernels do (`*d_position`, `*d_seq_len`: kernels/attention.cu:351, :1129),
 * instead of one entry per sequence. With batch 1 both conventions coincide.            */
#define HKV_FLAG_SCALAR_POSITION 1
/* The context only appends (hkv_append, hkv_append_at, hkv_qk_norm_rope_kv): no split-K or
 * prefill workspace is allocated; the attention entry points return HKV_ERR_WORKSPACE.  */
#define HKV_FLAG_APPEND_ONLY 2

typedef struct hkv_ctx hkv_ctx;

/* ---- lifetime ------------------------------------------------------------------- */

int hkv_abi_version(void);
const char* hkv_status_string(int status);

/* Validates the geometry and allocates the split-K workspace and the device status
 * word on the CURRENT device. Replaces nothing in the reference (its kernel needs no
 * workspace); the reference-side owner is the object that registers the ops
 * (kernels/register_kernels.cpp:649). */
int hkv_ctx_create(hkv_ctx** out, const hkv_geometry* geometry);
int hkv_ctx_destroy(hkv_ctx* ctx);
const char* hkv_ctx_last_error(const hkv_ctx* ctx);
/* Bytes of split-K workspace hkv_ctx_create allocates for this geometry. */
size_t hkv_workspace_bytes(const hkv_geometry* geometry);
/* Synchronises `stream`, reads the device status word and clears it. 0 = clean.
 * Non-zero bits: 1 = a bounded barrier wait ran out, 2 = an internal bound check failed. */
int hkv_ctx_device_status(hkv_ctx* ctx, void* stream, int32_t* status_out);
/* Which kernel the context selected: 1 = generic, 2 = TMA. */
int hkv_ctx_kernel(const hkv_ctx* ctx);
/* Kernels one decode call launches (for launch accounting). */
int hkv_ctx_launches_per_decode(const hkv_ctx* ctx);

/* ---- the path ------------------------------------------------------------------- */

/* KV append. Replaces launch_kv_cache_update_dp (kernels/attention.cu:1153-1170,
 * declared kernels/kernels.hpp:428-440) — K and V in one launch, 16-byte accesses.
 * d_cache_pos[b] is the write index of token 0 of sequence b: one entry PER SEQUENCE, where
 * the reference reads one scalar for the whole batch (HKV_FLAG_SCALAR_POSITION restores that). */
int hkv_append(hkv_ctx* ctx, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
               const int32_t* d_cache_pos, int32_t seq_new, void* stream);

/* Host-position twin. Replaces launch_kv_cache_update (kernels/attention.cu:1099-1116):
 * every sequence writes at `position`. */
int hkv_append_at(hkv_ctx* ctx, const void* k_new, const void* v_new, void* k_cache,
                  void* v_cache, int32_t position, int32_t seq_new, void* stream);

/* Cached decode attention. Replaces launch_attention_cached_fp16_dp
 * (kernels/attention.cu:496-510, declared kernels/kernels.hpp:468-482).
 * d_total_seq[b] = attended length (cache position + 1), one entry PER SEQUENCE (the reference
 * reads one scalar for the whole batch; HKV_FLAG_SCALAR_POSITION restores that). */
int hkv_decode_attention(hkv_ctx* ctx, const void* q, const void* k_cache, const void* v_cache,
                         void* out, const int32_t* d_total_seq, float scale, void* stream);

/* Host-length twin. Replaces launch_attention_cached_fp16 (kernels/attention.cu:318-334):
 * every sequence attends `seq_len` positions. The length travels as a kernel argument, so
 * back-to-back calls with different lengths need no synchronisation between them; a captured
 * graph freezes the length it was captured with. */
int hkv_decode_attention_len(hkv_ctx* ctx, const void* q, const void* k_cache,
                             const void* v_cache, void* out, int32_t seq_len, float scale,
                             void* stream);

/* Fused append + decode attention: the op the reference registry declares with five
 * inputs (Q, K_cache, V_cache, K_new, V_new; src/optype.cpp:118-120) but never
 * implements. Equals hkv_append(seq_new = 1) followed by hkv_decode_attention with
 * total = cache_pos + 1, in one pass over the cache. */
int hkv_append_decode_attention(hkv_ctx* ctx, const void* q, const void* k_new, const void* v_new,
                                void* k_cache, void* v_cache, void* out,
                                const int32_t* d_cache_pos, float scale, void* stream);

/* Prefill over the cache, batch 1 (a context of any other batch gets HKV_ERR_GEOMETRY).
 * Replaces launch_attention_prefill_cached_fp16 (kernels/attention.cu:775-788). The cache must
 * already hold the chunk. In a ring plane (HKV_LAYOUT_RING) the chunk must fit the plane together
 * with the window it attends: seq_new + window_size - 1 <= slots when past_len > 0. */
int hkv_prefill_attention(hkv_ctx* ctx, const void* q, const void* k_cache, const void* v_cache,
                          void* out, int32_t seq_new, int32_t past_len, float scale, void* stream);

/* Prefill chunk, append included: equals hkv_append_at(k_new, v_new at past_len) followed by
 * hkv_prefill_attention — the reference's KV_CACHE_UPDATE + ATTENTION_PREFILL_CACHED pair
 * (src/graph_builder.cpp emits them back to back; kernels/attention.cu:1099-1116, :775-788) — for
 * every plane, including a ring plane that cannot hold the chunk next to what it attends (a ring
 * of exactly window_size rows: the reference has no ring). There the chunk is attended BEFORE it
 * is appended, in two passes over the tensor cores — the rows already cached, and the chunk's own
 * k_new/v_new — whose partial rows are merged; then the rows are written. Needs window_size <=
 * slots, seq_new <= slots and, for that order, a context with max_seq_new >= seq_new.
 * k_new, v_new [seq_new, num_kv_heads, head_dim]; batch 1. */
int hkv_prefill_append_attention(hkv_ctx* ctx, const void* q, const void* k_new, const void* v_new,
                                 void* k_cache, void* v_cache, void* out, int32_t seq_new,
                                 int32_t past_len, float scale, void* stream);

/* Cached decode attention for callers that cannot allocate. It has no counterpart in the
 * reference. Same inputs, outputs and results as hkv_decode_attention, but it needs no
 * context: the split-K partials are kept in a fixed array inside the library image
 * instead of a cudaMalloc'ed workspace, and the call itself performs no cudaMalloc,
 * cudaFree or other allocating routine. It is meant for hosts that run under a memory
 * plan fixed at start-up (all HBM already given to the KV planes), for plugin sandboxes
 * that forbid allocation after initialisation, and for serving threads that cannot
 * accept the device-wide synchronisation an allocation implies.
 *   - Limit: batch * num_heads * (head_dim + 2) * 4 bytes must fit in
 *     HKV_STATIC_SCRATCH_BYTES (8 MiB); larger geometries get HKV_ERR_TOO_LARGE. Within
 *     that limit the split is coarsened automatically until the partials fit.
 *   - Every GPU that loads the library holds those 8 MiB until the process exits.
 *   - The first call on each device resolves the array's device address (set-up, no
 *     allocation); make that first call before any stream capture.
 *   - All calls on a device share the one array, which keeps the previous call's
 *     contents; nothing needs clearing between calls, but two calls that overlap on the
 *     GPU (different streams, or graphs replayed concurrently) race on it. Keep them on
 *     one stream or otherwise ordered.
 *   - Always runs the any-geometry SIMT kernel, so it is slower than a context. */
#define HKV_STATIC_SCRATCH_BYTES (8u << 20)
int hkv_decode_attention_static(const hkv_geometry* geometry, const void* q, const void* k_cache,
                                const void* v_cache, void* out, const int32_t* d_total_seq,
                                float scale, void* stream);

/* ---- sequence-split (multi-GPU) -------------------------------------------------- */

/* Floats per (sequence, head) in an exchanged partial: head_dim + 2  (o[], m, l). */
size_t hkv_partial_floats(const hkv_geometry* geometry);
/* Decode over this rank's shard of the cache; writes ONE merged fp32 partial per
 * (sequence, head) to `partial_out` [batch, num_heads, head_dim + 2]: un-normalised
 * output, running maximum (log2 domain) and sum. No counterpart in the reference
 * (it is single-GPU). k_new/v_new may be NULL (no append); otherwise the rank that
 * owns position d_cache_pos[b] appends it. */
int hkv_decode_partials(hkv_ctx* ctx, const void* q, const void* k_new, const void* v_new,
                        void* k_cache, void* v_cache, float* partial_out,
                        const int32_t* d_total_seq, float scale, void* stream);
/* Merge `num_parts` partials laid out [num_parts, batch, num_heads, head_dim + 2] (as an
 * all-gather delivers them) into fp16 `out`. */
int hkv_combine_partials(hkv_ctx* ctx, const float* partials, int32_t num_parts, void* out,
                         void* stream);

/* The same exchange WITHOUT a collective launch: the kernel that merges this rank's split-K
 * partials leaves the merged partial in this rank's own mailbox; the merge kernel first releases
 * it — an epoch flag stored into every rank's mailbox, one 4-byte store per rank over NVLink —
 * then waits, with a bound, for the flags of all ranks in its OWN mailbox and reads every rank's
 * partial straight from that rank's mailbox (plain peer loads over NVLink, no multicast) while it
 * merges. No counterpart in the reference (single-GPU).
 *
 * A mailbox is one device allocation of hkv_exchange_bytes() bytes per rank, zeroed once before
 * the first step, that every rank of the node has mapped (cudaIpcOpenMemHandle or any other peer
 * mapping): mailbox[r] is rank r's mailbox as THIS process addresses it, mailbox[rank] the local
 * one. Layout: 64 flag words (flag s = last epoch rank s has released), 64 state words of the owner
 * (its epoch counter and two CTA counters), then [2][batch*num_heads*(head_dim+2)] floats — the
 * owner's partial of two consecutive epochs, because a rank may run one exchange ahead of a peer that
 * is still merging the previous one. Every rank must make the same sequence of calls, each
 * hkv_decode_partials_publish followed by one hkv_merge_published on the same stream.
 *
 * hkv_decode_partials_publish: hkv_decode_partials with the mailbox as destination; never waits.
 * hkv_merge_published: releases, waits at most wait_limit_ms (0 = 2000) for every rank's flag, then
 *   writes fp16 `out` [batch, num_heads, head_dim], and closes the epoch. When the wait runs out the
 *   rows are left untouched, bit 1 of the device status word is set (hkv_ctx_device_status) and the
 *   kernel returns normally; later merges do not wait until the status word has been read.
 * Both only enqueue and are capturable; the epoch lives in the mailbox, so a captured pair can be
 * replayed. */
#define HKV_MAX_PEERS 8
typedef struct hkv_exchange {
    int32_t rank, world;             /* 0 <= rank < world <= HKV_MAX_PEERS                    */
    void* mailbox[HKV_MAX_PEERS];    /* 256-byte aligned; entries >= world are ignored          */
    int32_t wait_limit_ms;           /* bound of the merge kernel's wait; 0 = 2000, at most 10000 */
    int32_t reserved;
} hkv_exchange;
int hkv_exchange_bytes(const hkv_ctx* ctx, int32_t world, size_t* bytes_out);
int hkv_decode_partials_publish(hkv_ctx* ctx, const void* q, const void* k_new, const void* v_new,
                             void* k_cache, void* v_cache, const hkv_exchange* exchange,
                             const int32_t* d_total_seq, float scale, void* stream);
int hkv_merge_published(hkv_ctx* ctx, const hkv_exchange* exchange, void* out, void* stream);

/* ---- host-buffer convenience (end-to-end timing, tests) --------------------------- */

/* Fused op with HOST q / k_new / v_new / out (pinned memory recommended): copies the
 * inputs to context-owned device staging, runs hkv_append_decode_attention, copies the
 * result back; all on `stream`, no synchronisation. Not capturable. */
int hkv_append_decode_attention_host(hkv_ctx* ctx, const void* h_q, const void* h_k_new,
                                     const void* h_v_new, void* k_cache, void* v_cache,
                                     void* h_out, const int32_t* d_cache_pos, float scale,
                                     void* stream);

/* The same with the copies taken off `stream`: inputs go host -> device on a copy stream of the
 * context, the result device -> host on another, through a ring of four staging sets, so that the
 * copies of one call overlap the kernels of its neighbours (a decode step is one such call per
 * layer). Differences from the call above: the host inputs must be final when the call is MADE
 * (they are not ordered after earlier work on `stream`), and h_out is complete only once `stream`
 * has passed an hkv_host_flush enqueued after the call. The kernels themselves run on `stream` in
 * call order, so the cache planes see the same sequence of appends. Not capturable. */
int hkv_append_decode_attention_host_pipelined(hkv_ctx* ctx, const void* h_q, const void* h_k_new,
                                               const void* h_v_new, void* k_cache, void* v_cache,
                                               void* h_out, const int32_t* d_cache_pos, float scale,
                                               void* stream);
/* Makes `stream` wait for every output copy the pipelined call above has enqueued so far. */
int hkv_host_flush(hkv_ctx* ctx, void* stream);

/* ---- the step in front of the append (next row of the path) ------------------------ */

/* Per-head RMSNorm of q and k + rotary embedding; with cache planes given, the rotated K and
 * the V row are written straight into the cache at the device position (k itself is then left
 * untouched), so the separate append disappears. Replaces launch_qk_norm_rope_kv_fp16,
 * launch_qk_norm_rope_fp16 and launch_qk_norm_rope_fp16_dp (kernels/attention.cu:908-973,
 * declared kernels/kernels.hpp:331-352).
 *   q [batch, seq_new, num_heads, head_dim] in place; k, v [batch, seq_new, num_kv_heads, head_dim];
 *   q_norm_w, k_norm_w [head_dim]; k_cache / v_cache may both be NULL (then k is rewritten in
 *   place and v is ignored). Position of token s of sequence b = d_cache_pos[b] + s, or
 *   `position` + s when d_cache_pos is NULL. rotary_dim <= 0 means head_dim; scaling_factor <= 0
 *   means 1 (kernels/attention.cu:955-956). */
int hkv_qk_norm_rope_kv(hkv_ctx* ctx, void* q, void* k, const void* v, const void* q_norm_w,
                        const void* k_norm_w, void* k_cache, void* v_cache, const int32_t* d_cache_pos,
                        int32_t position, int32_t seq_new, int32_t rotary_dim, float eps, float theta,
                        float scaling_factor, void* stream);

/* ---- failure reporting self-test ---------------------------------------------------- */

/* Enqueues a one-warp kernel that waits, with the library's bounded wait, on a barrier that
 * nothing ever signals. After `limit_ms` (1..1000) the wait gives up, sets bit 1 of the
 * device status word and the kernel returns normally: hkv_ctx_device_status then reports
 * HKV_ERR_DEVICE_FAULT with status 1 and clears it, and the context stays usable. This is how
 * a lost producer inside the pipelined kernels surfaces: as a status, never as a hang or a
 * trap. No counterpart in the reference (its kernels have no device-side waits). */
int hkv_ctx_selftest_bounded_wait(hkv_ctx* ctx, int32_t limit_ms, void* stream);

/* ---- per-kernel timing (benchmarks; not capturable) -------------------------------- */

/* After hkv_ctx_profile_begin every decode call records CUDA events on its stream before
 * the split-K kernel, between it and the combine kernel, and after the combine kernel
 * (up to `max_calls` calls; later calls are not timed). hkv_ctx_profile_end synchronises
 * the stream, returns the summed durations in milliseconds and the number of timed
 * calls, and switches timing off. No counterpart in the reference at this level (its
 * Engine times whole ops, src/engine.cpp:299-316). */
int hkv_ctx_profile_begin(hkv_ctx* ctx, int32_t max_calls);
int hkv_ctx_profile_end(hkv_ctx* ctx, void* stream, float* decode_ms, float* combine_ms,
                        int32_t* calls);

/* ---- planning (host arithmetic only; works without a GPU) ------------------------- */

/* Row of this rank's plane that stores logical position `pos`, or -1 when the position
 * is not stored here (dropped past the end of a linear plane as in
 * kernels/attention.cu:1143-1144, or owned by another rank). */
int32_t hkv_slot_of_position(const hkv_geometry* geometry, int32_t pos);
/* Logical position held by row `slot` for a sequence of `total_seq` positions (may lie
 * outside the attended range). */
int32_t hkv_position_of_slot(const hkv_geometry* geometry, int32_t slot, int32_t total_seq);
/* Split-K plan of one sequence: first attended position, first 64-row tile, number of
 * tiles and number of work items (chunks) for `chunk_tiles` tiles per item. */
int hkv_plan_sequence(const hkv_geometry* geometry, int32_t total_seq, int32_t chunk_tiles,
                      int32_t* first_pos, int32_t* tile_lo, int32_t* n_tiles, int32_t* n_chunks);
/* The 64-row tiles the TMA decode kernel walks for a sequence of `total_seq` attended positions:
 * tile indices tile_lo, tile_lo + 1, ... (n_tiles of them), taken modulo *wrap_tiles when that is
 * non-zero — a wrapped ring plane larger than its window contributes only the cyclic run of tiles
 * its window touches. Host arithmetic only (tests, schedulers). */
int hkv_plan_decode_tiles(const hkv_geometry* geometry, int32_t total_seq, int32_t* tile_lo, int32_t* n_tiles,
                          int32_t* wrap_tiles);
/* The equal-span schedule of one decode launch, as the kernels derive it on the device: the tiles of
 * all sequences (host array totals[batch] of attended lengths) form one line of *total_tiles tiles cut
 * into *spans_used = min(spans_wanted, tiles) equal spans, span c covering tiles
 * [floor(T*c/S), floor(T*(c+1)/S)); sequence b's partials come from the spans
 * first_span[b] .. first_span[b] + n_parts[b] - 1 and sit at partial slot span + b. Host arithmetic only. */
int hkv_plan_decode_spans(const hkv_geometry* geometry, const int32_t* totals, int32_t spans_wanted,
                          int32_t* first_span, int32_t* n_parts, int32_t* total_tiles, int32_t* spans_used);

/* Plan of one hkv_prefill_attention call on a device with `sm_count` SMs (host arithmetic, no
 * device needed): query tiles in flight per CTA (2 or 1 for the tensor-core kernels, 0 = SIMT
 * kernel), number of work items, key-range splits per item and the shortest key span (in key
 * tiles: 128 rows, 64 for head_dim 256) of any item. splits <= min_span_tiles always holds: no
 * split is ever empty. *splits == 0 reports the equal-span schedule of the two-tile kernel (taken
 * whenever the context has a partial-row workspace for the chunk and no split count is forced):
 * all key tiles of all items form one line that is cut into *items equal spans, one per CTA, and an
 * item that straddles a cut is finished by the CTAs on either side (at most four per item). */
int hkv_plan_prefill(const hkv_geometry* geometry, int32_t seq_new, int32_t past_len, int32_t sm_count,
                     int32_t* tiles_in_flight, int32_t* items, int32_t* splits, int32_t* min_span_tiles);

/* Prefill chunk size (queries) at or below `target` for which the tensor-core kernel's work items
 * (pairs of query tiles x kv heads) are a whole multiple of `sm_count`: 2 * (128 / group) queries
 * per pair, pairs a multiple of sm_count / gcd(sm_count, num_kv_heads). With such a chunk no SM
 * idles in the last round of items (Qwen2-7B shape on 148 SMs: 1 332 or 2 664 queries run at
 * 1.2 PFLOP/s where 2 048 run at 1.0). Returns the smallest such size when `target` is below it,
 * `target` itself for geometries the tensor-core kernels do not take, <= 0 on bad arguments. */
int32_t hkv_preferred_prefill_chunk(const hkv_geometry* geometry, int32_t sm_count, int32_t target);

/* ---- utilities ------------------------------------------------------------------- */

/* Deterministic synthetic fp16 data, bit-identical to the CPU generator used by the
 * test oracle: element i gets value(seed, first_index + i), approximately N(0,1). */
int hkv_fill_synthetic(void* dst, uint64_t seed, uint64_t first_index, uint64_t count,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HKV_H_ */
