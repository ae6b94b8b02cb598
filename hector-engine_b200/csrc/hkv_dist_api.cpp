// hkv_dist_api.cpp — the C ABI of libhkv_dist (include/hkv_dist.h): a thin extern "C" shell over
// hkv::SeqSplitDecoder (host/hkv_seqsplit.hpp). Exceptions become status codes and a message.
#include <cstring>
#include <memory>
#include <new>
#include <string>

#include "../../include/hkv_dist.h"
#include "../host/hkv_seqsplit.hpp"

struct hkvd_decoder {
    std::unique_ptr<hkv::SeqSplitDecoder> dec;
    std::unique_ptr<hkv::NodeRoster> roster;
    std::string err;
};

namespace {
int fail(hkvd_decoder* d, int code, const std::string& msg) {
    if (d) d->err = msg;
    return code;
}
template <class F>
int guarded(hkvd_decoder* d, F&& f) {
    if (!d || !d->dec) return HKV_ERR_INVALID_ARG;
    try {
        return f();
    } catch (const std::exception& e) {
        const std::string what = e.what();
        const bool roster = what.find("step not launched") != std::string::npos;
        return fail(d, roster ? HKVD_ERR_ROSTER : HKVD_ERR_HOST, what);
    }
}
}  // namespace

extern "C" {

int hkvd_unique_id(void* out) {
    static_assert(sizeof(ncclUniqueId) == HKVD_UNIQUE_ID_BYTES, "ncclUniqueId size");
    if (!out) return HKV_ERR_INVALID_ARG;
    ncclUniqueId id;
    if (ncclGetUniqueId(&id) != ncclSuccess) return HKVD_ERR_HOST;
    std::memcpy(out, &id, sizeof id);
    return 0;
}

int hkvd_create(hkvd_decoder** out, const hkv_geometry* g, int32_t layers, const void* unique_id, float scale,
                void* stream) {
    return hkvd_create_with(out, g, layers, unique_id, scale, stream, HKVD_EXCHANGE_AUTO, 0);
}

int hkvd_create_with(hkvd_decoder** out, const hkv_geometry* g, int32_t layers, const void* unique_id, float scale,
                     void* stream, int32_t exchange, int32_t peer_wait_ms) {
    if (!out) return HKV_ERR_INVALID_ARG;
    *out = nullptr;
    hkvd_decoder* d = new (std::nothrow) hkvd_decoder();
    if (!d) return HKVD_ERR_HOST;
    *out = d;   // returned even on failure so that the caller can read the message; destroy it
    if (!g || layers <= 0) return fail(d, HKV_ERR_INVALID_ARG, "hkvd_create: null geometry or no layers");
    if (g->layout != HKV_LAYOUT_LINEAR || g->window_size != 0)
        return fail(d, HKV_ERR_GEOMETRY, "hkvd_create: sequence split takes linear planes without a window");
    if (g->q_seq_stride_elems != 0 || g->new_kv_seq_stride_elems != 0)
        return fail(d, HKV_ERR_GEOMETRY, "hkvd_create: the sequence-split step binds dense q / k_new / v_new (one block per layer)");
    hkv::SeqSplitConfig c;
    c.layers = (uint32_t)layers; c.batch = (uint32_t)g->batch; c.heads = (uint32_t)g->num_heads;
    c.kv_heads = (uint32_t)g->num_kv_heads; c.head_dim = (uint32_t)g->head_dim; c.local_slots = (uint32_t)g->slots;
    c.world = g->shard_count > 1 ? g->shard_count : 1;
    c.rank = g->shard_count > 1 ? g->shard_rank : 0;
    c.shard_block = g->shard_block > 0 ? (uint32_t)g->shard_block : 1024u;
    c.scale = scale; c.chunk_tiles = g->chunk_tiles; c.kernel_select = g->kernel_select;
    if (c.world > 1 && !unique_id) return fail(d, HKV_ERR_INVALID_ARG, "hkvd_create: shard_count > 1 needs a unique id");
    if (exchange < HKVD_EXCHANGE_AUTO || exchange > HKVD_EXCHANGE_PEER_STORES || peer_wait_ms < 0 || peer_wait_ms > 10000)
        return fail(d, HKV_ERR_INVALID_ARG, "hkvd_create: unknown exchange or wait limit outside 0..10000 ms");
    c.exchange = (hkv::Exchange)exchange;
    if (peer_wait_ms > 0) c.peer_wait_ms = peer_wait_ms;
    try {
        ncclUniqueId id;
        if (unique_id) std::memcpy(&id, unique_id, sizeof id);
        d->dec.reset(new hkv::SeqSplitDecoder(c, unique_id ? &id : nullptr, (cudaStream_t)stream));
    } catch (const std::exception& e) {
        return fail(d, HKVD_ERR_HOST, e.what());
    }
    return 0;
}

int hkvd_exchange(const hkvd_decoder* d, int32_t* exchange_out) {
    if (!d || !d->dec || !exchange_out) return HKV_ERR_INVALID_ARG;
    *exchange_out = (int32_t)d->dec->exchange();
    return 0;
}

int hkvd_destroy(hkvd_decoder* d) {
    if (!d) return 0;
    d->dec.reset();
    d->roster.reset();
    delete d;
    return 0;
}

const char* hkvd_last_error(const hkvd_decoder* d) { return d ? d->err.c_str() : "null decoder"; }

int hkvd_bind(hkvd_decoder* d, const void* q, const void* k_new, const void* v_new, void* out, void* k_planes,
              void* v_planes, uint64_t layer_stride_elems, const int32_t* d_total_seq) {
    return guarded(d, [&] {
        if (!q || !out || !k_planes || !v_planes || !d_total_seq || (k_new == nullptr) != (v_new == nullptr))
            return fail(d, HKV_ERR_INVALID_ARG, "hkvd_bind: null tensor (k_new and v_new go together)");
        d->dec->bind((const half*)q, (const half*)k_new, (const half*)v_new, (half*)out, (half*)k_planes, (half*)v_planes,
                     (size_t)layer_stride_elems, d_total_seq);
        return 0;
    });
}

int hkvd_step(hkvd_decoder* d, int32_t mode, int32_t* replayed) {
    return guarded(d, [&] {
        bool r = false;
        if (mode == 0) r = d->dec->step();
        else d->dec->step_eager();
        if (replayed) *replayed = r ? 1 : 0;
        return 0;
    });
}

int hkvd_step_profiled(hkvd_decoder* d, float* decode_ms, float* gather_ms, float* combine_ms) {
    return guarded(d, [&] {
        const hkv::SeqSplitTimes t = d->dec->step_profiled();
        if (decode_ms) *decode_ms = t.decode_ms;
        if (gather_ms) *gather_ms = t.gather_ms;
        if (combine_ms) *combine_ms = t.combine_ms;
        return 0;
    });
}

int hkvd_wait(hkvd_decoder* d, int32_t timeout_ms) {
    return guarded(d, [&] {
        if (timeout_ms < 0) return fail(d, HKV_ERR_INVALID_ARG, "hkvd_wait: negative timeout");
        const hkv::WatchResult r = d->dec->wait(std::chrono::milliseconds(timeout_ms));
        if (r == hkv::WatchResult::Done) return 0;
        return fail(d, r == hkv::WatchResult::PeerError ? HKVD_ERR_PEER : HKVD_ERR_TIMEOUT, hkv::watch_result_name(r));
    });
}

int hkvd_device_status(hkvd_decoder* d, int32_t* status_out) {
    return guarded(d, [&] {
        if (!status_out) return (int)HKV_ERR_INVALID_ARG;
        *status_out = d->dec->device_status();
        return *status_out ? (int)HKV_ERR_DEVICE_FAULT : 0;
    });
}

int hkvd_attach_roster(hkvd_decoder* d, const char* name, int32_t fresh, int32_t grace_ms) {
    return guarded(d, [&] {
        if (!name || grace_ms < 0) return fail(d, HKV_ERR_INVALID_ARG, "hkvd_attach_roster: bad arguments");
        d->roster.reset(new hkv::NodeRoster(name, d->dec->config().world, d->dec->config().rank, fresh != 0));
        d->dec->attach_roster(d->roster.get(), std::chrono::milliseconds(grace_ms));
        return 0;
    });
}

int hkvd_leave(hkvd_decoder* d) {
    return guarded(d, [&] {
        if (!d->roster) return fail(d, HKV_ERR_INVALID_ARG, "hkvd_leave: no roster attached");
        d->roster->leave();
        return 0;
    });
}

}  // extern "C"
