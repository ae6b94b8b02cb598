// hkv_seqsplit.hpp — sequence-split decode over the GPUs of one node, hosted in C++.
//
// One logical KV cache per sequence is dealt block-cyclically over `world` ranks (one process per
// GPU): logical block j of `shard_block` positions lives on rank j % world as local block j / world
// (hkv_geometry.shard_*). Per layer, on the compute stream:
//     hkv_decode_partials     split-K decode over THIS rank's rows, one fp32 partial
//                             (o[head_dim], m, l) per (sequence, head); the rank that owns the new
//                             token's position stages and stores its K/V row inside the same kernel
//     ncclAllGather           batch*heads*(head_dim+2)*4 bytes per rank, NVLink/NVSwitch
//     hkv_combine_partials    merges the `world` partials, fp16 output replicated on every rank
// or, when every rank can map every other rank's memory (Exchange::PeerStores, the default then),
// without any collective launch:
//     hkv_decode_partials_publish  the same decode; the kernel that merges this rank's split-K partials
//                                  leaves the result in this rank's mailbox
//     hkv_merge_published          releases it (an epoch flag into every rank's mailbox: 4-byte stores
//                                  over NVLink), waits — bounded — for all flags in its OWN mailbox, then
//                                  reads every rank's partial from that rank's mailbox (plain peer
//                                  loads) while it merges, writes fp16
// Mailboxes are cudaMalloc'd per rank and mapped by the others through CUDA IPC handles, handed
// round once at construction with an NCCL all-gather. The only cross-GPU wait is the merge kernel's
// bounded poll of flag words in local memory.
// The whole multi-layer step is captured ONCE into a CUDA graph (NCCL collectives and the mailbox
// kernels are capturable: the epoch lives in device memory) and replayed while only the device-side
// length array changes, under the same capture rules as the engine's own graph (reference
// src/engine.cpp:206-231: work only on the capture stream, no allocation, no synchronisation, no
// host reads).
//
// Failure handling is host-side (hkv_step_watch.hpp): wait() polls the stream and
// ncclCommGetAsyncError against a deadline and aborts the communicator when a peer is stuck or
// gone; in mailbox mode a peer that stops pushing makes the merge kernel's wait run out (status
// word, the kernel returns), which wait() reports as TimedOut; an optional NodeRoster lets a rank
// that left between steps be noticed before the launch.
//
// The reference engine has no multi-GPU path (its README lists it as absent); this is new work
// behind the same C ABI (include/hkv.h).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nccl.h>

#include <chrono>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "hkv.h"
#include "hkv_decode_loop.hpp"
#include "hkv_step_watch.hpp"

namespace hkv {

enum class Exchange : int32_t {
    Auto = 0,        // PeerStores when every rank managed to map every mailbox, else Nccl
    Nccl = 1,        // ncclAllGather between the two kernels
    PeerStores = 2,  // mailboxes (peer-mapped memory); construction fails when a mapping is refused
};

struct SeqSplitConfig {
    uint32_t layers = 0, batch = 1, heads = 0, kv_heads = 0, head_dim = 0;
    uint32_t local_slots = 0;    // rows per sequence held by THIS rank
    uint32_t shard_block = 1024; // positions per dealt block (multiple of 64)
    int rank = 0, world = 1;
    float scale = 0.0f;          // 0 = 1/sqrt(head_dim) (reference default, src/command.cpp:160)
    int32_t chunk_tiles = 0, kernel_select = 0;
    Exchange exchange = Exchange::Auto;
    int32_t peer_wait_ms = 2000;  // bound of the merge kernel's wait for the peers' flags
};

struct SeqSplitTimes {
    float decode_ms = 0, gather_ms = 0, combine_ms = 0;   // summed over the layers of one step
};

class SeqSplitDecoder {
public:
    // `id` is the communicator's unique id (ncclGetUniqueId on one rank, handed to the others by
    // the launcher's own means); ignored when world == 1. Allocates: construct before any capture.
    SeqSplitDecoder(const SeqSplitConfig& cfg, const ncclUniqueId* id, cudaStream_t stream)
        : cfg_(cfg), stream_(stream) {
        try {
            construct(id);
        } catch (...) {
            release(false);   // a constructor that throws runs no destructor: give back what it took
            throw;
        }
    }
    ~SeqSplitDecoder() { release(true); }
    SeqSplitDecoder(const SeqSplitDecoder&) = delete;
    SeqSplitDecoder& operator=(const SeqSplitDecoder&) = delete;

    const SeqSplitConfig& config() const { return cfg_; }
    hkv_ctx* context() { return ctx_; }
    GraphReplay& graph() { return graph_; }
    uint64_t steps() const { return steps_; }
    size_t partial_bytes() const { return part_floats_ * sizeof(float); }
    // What moves the partials between the ranks (decided at construction, the same on every rank).
    Exchange exchange() const { return peer_ ? Exchange::PeerStores : Exchange::Nccl; }

    // Buffers the step reads and writes; they keep their addresses for as long as the graph lives
    // (rebinding drops it). Per layer l:
    //   q + l*batch*heads*head_dim, k_new/v_new + l*batch*kv_heads*head_dim, out like q,
    //   k_planes/v_planes + l*layer_stride_elems  ([batch][local_slots][kv_heads][head_dim] each).
    // k_new/v_new may be null (attention only). d_total_seq[b] = attended length of sequence b in
    // LOGICAL positions (the new token included), identical on every rank.
    void bind(const half* q, const half* k_new, const half* v_new, half* out, half* k_planes, half* v_planes,
              size_t layer_stride_elems, const int32_t* d_total_seq) {
        q_ = q; k_new_ = k_new; v_new_ = v_new; out_ = out; k_ = k_planes; v_ = v_planes;
        layer_stride_ = layer_stride_elems; d_total_ = d_total_seq;
        graph_.invalidate();
    }
    void attach_roster(NodeRoster* roster, std::chrono::milliseconds grace = std::chrono::milliseconds(1000)) {
        roster_ = roster;
        grace_ = grace;
    }

    // One token for every sequence: all layers, captured once and replayed. Only enqueues. Returns
    // true when the step was a graph replay. With a roster attached the step is announced and the
    // peers are checked first; a peer that left or fell behind throws BEFORE anything is enqueued.
    bool step() {
        require_bound();
        pre_launch();
        // The first step runs un-captured, as the engine's first token does: NCCL sets up its
        // channels (and allocates) on a communicator's first collective, which must not happen
        // inside a capture.
        if (!warmed_) {
            enqueue_layers(stream_, nullptr);
            warmed_ = true;
            ++steps_;
            return false;
        }
        const bool replayed = graph_.run(stream_, [this](cudaStream_t s) { enqueue_layers(s, nullptr); });
        ++steps_;
        return replayed;
    }
    // The same step enqueued call by call (no graph).
    void step_eager() {
        require_bound();
        pre_launch();
        enqueue_layers(stream_, nullptr);
        warmed_ = true;
        ++steps_;
    }
    // The same step with CUDA events around every phase of every layer; synchronises the stream.
    SeqSplitTimes step_profiled() {
        require_bound();
        pre_launch();
        while (events_.size() < (size_t)cfg_.layers * 4) {
            cudaEvent_t e;
            cuda_check(cudaEventCreate(&e), "cudaEventCreate");
            events_.push_back(e);
        }
        enqueue_layers(stream_, events_.data());
        warmed_ = true;
        ++steps_;
        cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
        SeqSplitTimes t;
        for (uint32_t l = 0; l < cfg_.layers; ++l) {
            float a = 0, b = 0, c = 0;
            cudaEventElapsedTime(&a, events_[l * 4], events_[l * 4 + 1]);
            cudaEventElapsedTime(&b, events_[l * 4 + 1], events_[l * 4 + 2]);
            cudaEventElapsedTime(&c, events_[l * 4 + 2], events_[l * 4 + 3]);
            t.decode_ms += a; t.gather_ms += b; t.combine_ms += c;
        }
        return t;
    }

    // Host-side wait for everything enqueued so far, with a deadline. On PeerError / TimedOut the
    // communicator is aborted (its pending collectives are cancelled; the object then only serves
    // destruction). Never blocks longer than `timeout`.
    WatchResult wait(std::chrono::milliseconds timeout) {
        const WatchResult r = watch_step(
            [this] { return cudaStreamQuery(stream_) == cudaSuccess; },
            [this] {
                if (!comm_) return false;
                ncclResult_t async = ncclSuccess;
                return ncclCommGetAsyncError(comm_, &async) != ncclSuccess || (async != ncclSuccess && async != ncclInProgress);
            },
            timeout);
        if (r != WatchResult::Done && comm_ && !aborted_) abandon();
        cudaGetLastError();
        if (r == WatchResult::Done && peer_ && (device_status() & 1)) {
            // a merge kernel gave up waiting for a peer's flag: the step's output is not valid
            if (!aborted_) abandon();
            return WatchResult::TimedOut;
        }
        return r;
    }
    // Tears the communicator down without the peers (ncclCommAbort): for a rank that leaves, and
    // for the ranks it leaves behind. Call with nothing of this rank in flight. The object then
    // only serves destruction.
    void abandon() {
        // The captured graph goes first: a graph that holds this communicator's collectives keeps the
        // communicator referenced, and NCCL's abort (like its destroy) waits for those references.
        graph_.invalidate();
        if (comm_) ncclCommAbort(comm_);
        comm_ = nullptr;
        aborted_ = true;
    }
    bool aborted() const { return aborted_; }
    int device_status() { int32_t w = 0; hkv_ctx_device_status(ctx_, stream_, &w); return w; }

private:
    void construct(const ncclUniqueId* id) {
        const SeqSplitConfig& cfg = cfg_;
        if (!cfg.layers || !cfg.batch || !cfg.heads || !cfg.kv_heads || !cfg.head_dim || !cfg.local_slots)
            throw std::runtime_error("SeqSplitDecoder: incomplete configuration");
        if (cfg.world < 1 || cfg.rank < 0 || cfg.rank >= cfg.world)
            throw std::runtime_error("SeqSplitDecoder: rank/world out of range");
        if (cfg_.scale == 0.0f) cfg_.scale = 1.0f / std::sqrt((float)cfg.head_dim);
        hkv_geometry g{};
        g.batch = (int32_t)cfg.batch; g.num_heads = (int32_t)cfg.heads; g.num_kv_heads = (int32_t)cfg.kv_heads;
        g.head_dim = (int32_t)cfg.head_dim; g.slots = (int32_t)cfg.local_slots; g.layout = HKV_LAYOUT_LINEAR;
        g.shard_rank = cfg.rank; g.shard_count = cfg.world; g.shard_block = (int32_t)cfg.shard_block;
        g.chunk_tiles = cfg.chunk_tiles; g.kernel_select = cfg.kernel_select;
        const int st = hkv_ctx_create(&ctx_, &g);
        if (st != HKV_OK) {
            std::string msg = std::string("SeqSplitDecoder: hkv_ctx_create: ") + hkv_status_string(st);
            if (ctx_) msg += std::string(" (") + hkv_ctx_last_error(ctx_) + ")";
            throw std::runtime_error(msg);
        }
        part_floats_ = (size_t)cfg.batch * cfg.heads * (cfg.head_dim + 2);
        cuda_check(cudaMalloc(&part_, part_floats_ * sizeof(float)), "cudaMalloc(partial)");
        cuda_check(cudaMalloc(&gathered_, part_floats_ * sizeof(float) * cfg.world), "cudaMalloc(gathered)");
        if (cfg.world > 1) {
            if (!id) throw std::runtime_error("SeqSplitDecoder: world > 1 needs a communicator id");
            const ncclResult_t r = ncclCommInitRank(&comm_, cfg.world, *id, cfg.rank);
            if (r != ncclSuccess) throw std::runtime_error(std::string("SeqSplitDecoder: ncclCommInitRank: ") + ncclGetErrorString(r));
            if (cfg.exchange != Exchange::Nccl) {
                if (cfg.world > HKV_MAX_PEERS) {
                    if (cfg.exchange == Exchange::PeerStores)
                        throw std::runtime_error("SeqSplitDecoder: mailboxes serve at most " + std::to_string(HKV_MAX_PEERS) + " ranks");
                } else {
                    std::string why;
                    peer_ = map_mailboxes(&why);
                    if (!peer_ && cfg.exchange == Exchange::PeerStores)
                        throw std::runtime_error("SeqSplitDecoder: mailboxes could not be mapped on every rank: " + why);
                }
            }
        }
    }
    // Gives everything back. `meet`: the ranks are torn down together (the destructor of a healthy decoder).
    void release(bool meet) {
        graph_.invalidate();
        cudaStreamSynchronize(stream_);
        // A peer may still be reading this rank's last partial (its merge of the last step): the ranks
        // meet once more before any mailbox is freed — unless the communicator is gone, in which case
        // the peers have stopped launching (a departure is announced between steps).
        if (meet && peer_ && comm_ && !aborted_ && meet_ != nullptr &&
            ncclAllReduce(meet_, meet_, 1, ncclInt, ncclSum, comm_, stream_) == ncclSuccess) {
            // with a deadline: a rank that is torn down alone (an error path) must not wait for ever
            const WatchResult met = watch_step([this] { return cudaStreamQuery(stream_) == cudaSuccess; },
                                               [] { return false; }, std::chrono::milliseconds(5000));
            if (met != WatchResult::Done) {
                ncclCommAbort(comm_);
                comm_ = nullptr;
            }
        }
        unmap_mailboxes();
        if (meet_) cudaFree(meet_);
        meet_ = nullptr;
        for (cudaEvent_t e : events_) cudaEventDestroy(e);
        events_.clear();
        if (comm_) (meet ? ncclCommDestroy(comm_) : ncclCommAbort(comm_));
        comm_ = nullptr;
        if (part_) cudaFree(part_);
        if (gathered_) cudaFree(gathered_);
        part_ = gathered_ = nullptr;
        if (ctx_) hkv_ctx_destroy(ctx_);
        ctx_ = nullptr;
    }
    static void cuda_check(cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string("SeqSplitDecoder: ") + what + ": " + cudaGetErrorString(e));
    }
    void require_bound() const {
        if (!q_ || !out_ || !k_ || !v_ || !d_total_) throw std::runtime_error("SeqSplitDecoder: bind() first");
        if (aborted_) throw std::runtime_error("SeqSplitDecoder: the communicator was aborted");
    }
    void pre_launch() {
        if (!roster_) return;
        roster_->announce(steps_ + 1);
        int who = -1;
        const NodeRoster::Check c = roster_->check_before_launch(steps_ + 1, grace_, &who);
        if (c == NodeRoster::Check::PeerLeft)
            throw std::runtime_error("SeqSplitDecoder: rank " + std::to_string(who) + " has left; step not launched");
        if (c == NodeRoster::Check::PeerBehind)
            throw std::runtime_error("SeqSplitDecoder: rank " + std::to_string(who) + " is not keeping up; step not launched");
    }
    void hkv_check(int st, const char* what, uint32_t layer) const {
        if (st != HKV_OK)
            throw std::runtime_error(std::string("SeqSplitDecoder: ") + what + " (layer " + std::to_string(layer) + "): " +
                                     hkv_ctx_last_error(ctx_));
    }
    // Allocates and zeroes this rank's mailbox, hands its IPC handle round (one NCCL all-gather, which
    // also orders every rank's zeroing before anybody's first push) and maps the others'. Returns
    // whether EVERY rank succeeded (agreed by an all-reduce), so that all ranks pick the same exchange.
    bool map_mailboxes(std::string* why) {
        const int world = cfg_.world, rank = cfg_.rank;
        bool ok = true;
        size_t bytes = 0;
        if (hkv_exchange_bytes(ctx_, world, &bytes) != HKV_OK) { ok = false; *why = "hkv_exchange_bytes"; }
        cudaIpcMemHandle_t mine{};
        if (cudaMalloc(&meet_, sizeof(int)) != cudaSuccess || cudaMemset(meet_, 0, sizeof(int)) != cudaSuccess) {
            ok = false;
            *why = "cudaMalloc(meeting word)";
        }
        if (ok && (cudaMalloc(&mailbox_, bytes) != cudaSuccess || cudaMemset(mailbox_, 0, bytes) != cudaSuccess ||
                   cudaDeviceSynchronize() != cudaSuccess || cudaIpcGetMemHandle(&mine, mailbox_) != cudaSuccess)) {
            ok = false;
            *why = std::string("mailbox allocation / cudaIpcGetMemHandle: ") + cudaGetErrorString(cudaGetLastError());
        }
        // handles (and a success flag per rank) travel in one device buffer
        constexpr size_t kSlot = sizeof(cudaIpcMemHandle_t) + 8;
        std::vector<unsigned char> host(kSlot * world, 0);
        unsigned char* d_all = nullptr;
        cuda_check(cudaMalloc(&d_all, kSlot * world), "cudaMalloc(handles)");
        std::memcpy(host.data() + kSlot * rank, &mine, sizeof mine);
        host[kSlot * rank + sizeof mine] = ok ? 1 : 0;
        cuda_check(cudaMemcpy(d_all + kSlot * rank, host.data() + kSlot * rank, kSlot, cudaMemcpyHostToDevice), "cudaMemcpy(handle)");
        ncclResult_t r = ncclAllGather(d_all + kSlot * rank, d_all, kSlot, ncclChar, comm_, stream_);
        if (r != ncclSuccess) { cudaFree(d_all); throw std::runtime_error(std::string("SeqSplitDecoder: ncclAllGather(handles): ") + ncclGetErrorString(r)); }
        cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize(handles)");
        cuda_check(cudaMemcpy(host.data(), d_all, kSlot * world, cudaMemcpyDeviceToHost), "cudaMemcpy(handles)");
        for (int p = 0; p < world; ++p) ok = ok && host[kSlot * p + sizeof mine] == 1;
        x_ = hkv_exchange{};
        x_.rank = rank; x_.world = world; x_.wait_limit_ms = cfg_.peer_wait_ms;
        if (ok) {
            for (int p = 0; p < world && ok; ++p) {
                if (p == rank) { x_.mailbox[p] = mailbox_; continue; }
                cudaIpcMemHandle_t h;
                std::memcpy(&h, host.data() + kSlot * p, sizeof h);
                void* mapped = nullptr;
                const cudaError_t e = cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess);
                if (e != cudaSuccess) {
                    ok = false;
                    *why = "cudaIpcOpenMemHandle(rank " + std::to_string(p) + "): " + cudaGetErrorString(e);
                    cudaGetLastError();
                } else {
                    x_.mailbox[p] = mapped;
                }
            }
        }
        // agree: one byte per rank again
        std::fill(host.begin(), host.end(), 0);
        host[kSlot * rank] = ok ? 1 : 0;
        cuda_check(cudaMemcpy(d_all + kSlot * rank, host.data() + kSlot * rank, kSlot, cudaMemcpyHostToDevice), "cudaMemcpy(agree)");
        r = ncclAllGather(d_all + kSlot * rank, d_all, kSlot, ncclChar, comm_, stream_);
        if (r != ncclSuccess) { cudaFree(d_all); throw std::runtime_error(std::string("SeqSplitDecoder: ncclAllGather(agree): ") + ncclGetErrorString(r)); }
        cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize(agree)");
        cuda_check(cudaMemcpy(host.data(), d_all, kSlot * world, cudaMemcpyDeviceToHost), "cudaMemcpy(agree)");
        cudaFree(d_all);
        bool all = true;
        for (int p = 0; p < world; ++p)
            if (host[kSlot * p] != 1) { all = false; if (why->empty()) *why = "rank " + std::to_string(p) + " could not map a mailbox"; }
        if (!all) unmap_mailboxes();
        return all;
    }
    void unmap_mailboxes() {
        for (int p = 0; p < HKV_MAX_PEERS; ++p) {
            if (p != cfg_.rank && x_.mailbox[p]) cudaIpcCloseMemHandle(x_.mailbox[p]);
            x_.mailbox[p] = nullptr;
        }
        if (mailbox_) cudaFree(mailbox_);
        mailbox_ = nullptr;
        peer_ = false;
    }
    void enqueue_layers(cudaStream_t s, cudaEvent_t* ev) {
        const size_t qn = (size_t)cfg_.batch * cfg_.heads * cfg_.head_dim;
        const size_t kn = (size_t)cfg_.batch * cfg_.kv_heads * cfg_.head_dim;
        for (uint32_t l = 0; l < cfg_.layers && peer_; ++l) {
            if (ev) cudaEventRecord(ev[l * 4], s);
            hkv_check(hkv_decode_partials_publish(ctx_, q_ + l * qn, k_new_ ? k_new_ + l * kn : nullptr,
                                               v_new_ ? v_new_ + l * kn : nullptr, k_ + l * layer_stride_,
                                               v_ + l * layer_stride_, &x_, d_total_, cfg_.scale, s),
                      "hkv_decode_partials_publish", l);
            if (ev) { cudaEventRecord(ev[l * 4 + 1], s); cudaEventRecord(ev[l * 4 + 2], s); }
            hkv_check(hkv_merge_published(ctx_, &x_, out_ + l * qn, s), "hkv_merge_published", l);
            if (ev) cudaEventRecord(ev[l * 4 + 3], s);
        }
        if (peer_) return;
        for (uint32_t l = 0; l < cfg_.layers; ++l) {
            if (ev) cudaEventRecord(ev[l * 4], s);
            hkv_check(hkv_decode_partials(ctx_, q_ + l * qn, k_new_ ? k_new_ + l * kn : nullptr,
                                          v_new_ ? v_new_ + l * kn : nullptr, k_ + l * layer_stride_, v_ + l * layer_stride_,
                                          part_, d_total_, cfg_.scale, s),
                      "hkv_decode_partials", l);
            if (ev) cudaEventRecord(ev[l * 4 + 1], s);
            const float* merged = part_;
            if (comm_) {
                const ncclResult_t r = ncclAllGather(part_, gathered_, part_floats_, ncclFloat, comm_, s);
                if (r != ncclSuccess) throw std::runtime_error(std::string("SeqSplitDecoder: ncclAllGather: ") + ncclGetErrorString(r));
                merged = gathered_;
            }
            if (ev) cudaEventRecord(ev[l * 4 + 2], s);
            hkv_check(hkv_combine_partials(ctx_, merged, comm_ ? cfg_.world : 1, out_ + l * qn, s), "hkv_combine_partials", l);
            if (ev) cudaEventRecord(ev[l * 4 + 3], s);
        }
    }

    SeqSplitConfig cfg_;
    cudaStream_t stream_;
    hkv_ctx* ctx_ = nullptr;
    ncclComm_t comm_ = nullptr;
    bool aborted_ = false;
    bool warmed_ = false;   // a collective has run outside capture
    float* part_ = nullptr;       // [batch][heads][head_dim + 2]
    float* gathered_ = nullptr;   // [world][batch][heads][head_dim + 2]
    bool peer_ = false;           // partials travel through mailboxes, not a collective
    void* mailbox_ = nullptr;     // this rank's mailbox (hkv_exchange_bytes)
    int* meet_ = nullptr;         // one word for the all-reduce the ranks meet on before mailboxes are freed
    hkv_exchange x_{};            // every rank's mailbox as mapped here
    size_t part_floats_ = 0;
    GraphReplay graph_;
    std::vector<cudaEvent_t> events_;
    NodeRoster* roster_ = nullptr;
    std::chrono::milliseconds grace_{1000};
    const half* q_ = nullptr;
    const half* k_new_ = nullptr;
    const half* v_new_ = nullptr;
    half* out_ = nullptr;
    half* k_ = nullptr;
    half* v_ = nullptr;
    size_t layer_stride_ = 0;
    const int32_t* d_total_ = nullptr;
    uint64_t steps_ = 0;
};

}  // namespace hkv
