/* hkv_dist.h — C ABI of libhkv_dist: the sequence-split decode step over the GPUs of one node
 * (one process per GPU), hosted in C++ over libhkv's kernels and NCCL.
 *
 * None of these entry points has a counterpart in the reference engine, which is single-GPU
 * (its README lists multi-GPU as absent); they sit behind the same boundary as include/hkv.h so
 * that an engine process per GPU can drive long-context decode.
 *
 * Per layer the step is  hkv_decode_partials -> ncclAllGather -> hkv_combine_partials  (or, without a
 * collective launch, hkv_decode_partials_publish -> hkv_merge_published through peer-mapped mailboxes) on the
 * caller's stream; hkvd_step captures all layers once into a CUDA graph and replays it while only
 * the device-side length array changes. Every function returns 0 on success, an hkv_status
 * (include/hkv.h) or HKVD_* below otherwise; hkvd_last_error gives the text. Nothing here waits
 * on a GPU without a deadline.
 */
#ifndef HKV_DIST_H_
#define HKV_DIST_H_

#include <stddef.h>
#include <stdint.h>

#include "hkv.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HKVD_UNIQUE_ID_BYTES 128
#define HKVD_ERR_PEER 101     /* the communicator reported an asynchronous error; it was aborted  */
#define HKVD_ERR_TIMEOUT 102  /* the step did not finish before the deadline; communicator aborted */
#define HKVD_ERR_ROSTER 103   /* a peer left or fell behind: the step was NOT launched             */
#define HKVD_ERR_HOST 104     /* any other host-side failure (message in hkvd_last_error)          */

typedef struct hkvd_decoder hkvd_decoder;

/* Fills `out` (HKVD_UNIQUE_ID_BYTES) with a fresh communicator id (ncclGetUniqueId). Call on one
 * rank and hand the bytes to the others by the launcher's own means. */
int hkvd_unique_id(void* out);

/* Creates this rank's decoder on the CURRENT device: context, partial buffers, communicator.
 * `geometry` describes THIS rank's planes: slots = rows per sequence held here; shard_rank,
 * shard_count, shard_block describe the block-cyclic deal; layout linear. `unique_id` may be NULL
 * when shard_count <= 1. Allocates and initialises NCCL: not capturable; collective over all ranks. */
int hkvd_create(hkvd_decoder** out, const hkv_geometry* geometry, int32_t layers, const void* unique_id,
                float scale, void* stream);
/* The same with the exchange chosen by the caller. HKVD_EXCHANGE_NCCL: ncclAllGather between the two
 * kernels of a layer. HKVD_EXCHANGE_PEER_STORES: no collective launch — each rank's partial-merging
 * kernel publishes an epoch flag in every rank's mailbox over NVLink and the final merge reads the
 * ranks' partials through the peer-mapped mailboxes (hkv_decode_partials_publish / hkv_merge_published,
 * include/hkv.h); needs every rank to map every other rank's mailbox through CUDA IPC (one process per
 * GPU on one node, at most HKV_MAX_PEERS ranks) and fails otherwise. HKVD_EXCHANGE_AUTO (what hkvd_create
 * uses): peer stores when every rank could map, else NCCL; all ranks always agree. peer_wait_ms bounds
 * the merge kernel's wait for the peers' flags (0 = 2000); when it runs out hkvd_wait returns
 * HKVD_ERR_TIMEOUT. hkvd_exchange reports what the decoder uses. */
#define HKVD_EXCHANGE_AUTO 0
#define HKVD_EXCHANGE_NCCL 1
#define HKVD_EXCHANGE_PEER_STORES 2
int hkvd_create_with(hkvd_decoder** out, const hkv_geometry* geometry, int32_t layers, const void* unique_id,
                     float scale, void* stream, int32_t exchange, int32_t peer_wait_ms);
int hkvd_exchange(const hkvd_decoder* d, int32_t* exchange_out);
int hkvd_destroy(hkvd_decoder* d);
const char* hkvd_last_error(const hkvd_decoder* d);

/* Binds the buffers of the step (fixed addresses while the graph lives). Layer l reads
 * q + l*batch*heads*head_dim, k_new/v_new + l*batch*kv_heads*head_dim (either may be NULL: no
 * append), the planes at k_planes/v_planes + l*layer_stride_elems, and writes out like q.
 * d_total_seq[b] = attended length in LOGICAL positions, identical on every rank. */
int hkvd_bind(hkvd_decoder* d, const void* q, const void* k_new, const void* v_new, void* out, void* k_planes,
              void* v_planes, uint64_t layer_stride_elems, const int32_t* d_total_seq);

/* Enqueues one step on the decoder's stream. mode 0: captured graph (the first call runs
 * un-captured so that NCCL can set up outside capture, the second captures); mode 1: call by call.
 * *replayed (may be NULL) = 1 when the step was a graph replay. */
int hkvd_step(hkvd_decoder* d, int32_t mode, int32_t* replayed);
/* One step with CUDA events around each phase of each layer; synchronises. Sums over layers, ms. */
int hkvd_step_profiled(hkvd_decoder* d, float* decode_ms, float* gather_ms, float* combine_ms);
/* Host-side wait, at most `timeout_ms`: 0 when everything enqueued has completed; HKVD_ERR_PEER or
 * HKVD_ERR_TIMEOUT after aborting the communicator (the decoder can then only be destroyed). */
int hkvd_wait(hkvd_decoder* d, int32_t timeout_ms);
/* Device status word of the decoder's context (see hkv_ctx_device_status); synchronises. */
int hkvd_device_status(hkvd_decoder* d, int32_t* status_out);

/* Optional roster of the node's ranks in POSIX shared memory (`name` like "/hkv-job42", the same
 * on every rank; rank 0 passes fresh = 1 and must open it first). With a roster, hkvd_step first
 * announces the step and checks the peers: if one has left or is more than a step behind after
 * `grace_ms`, HKVD_ERR_ROSTER is returned and nothing is enqueued. hkvd_leave marks this rank as
 * gone; call it between steps, with nothing of this rank in flight. */
int hkvd_attach_roster(hkvd_decoder* d, const char* name, int32_t fresh, int32_t grace_ms);
int hkvd_leave(hkvd_decoder* d);

#ifdef __cplusplus
}
#endif
#endif /* HKV_DIST_H_ */
