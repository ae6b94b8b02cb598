// hkv_seqsplit_tests.cpp — C++ test of hkv::SeqSplitDecoder (host/hkv_seqsplit.hpp): the
// sequence-split decode step, one process per GPU, NCCL all-gather of the partials on the compute
// stream, the whole multi-layer step captured once and replayed. Checked against the CPU oracle on
// the full logical cache; the rank that owns a new token's position must hold its row bit-exact.
//
//   hkv_seqsplit_tests                 parent: picks world = min(GPUs, 4); world 1 runs in-process,
//                                      otherwise spawns one child per GPU and waits (with a limit)
//   hkv_seqsplit_tests --rank r --world w --idfile f [--leave]     one rank
//
// With --leave (only given when world >= 2) the last rank leaves after the checked steps, between
// steps and with nothing in flight; the others must learn of it from the roster on the host and
// refuse the next step before launching anything. No GPU is made to wait, fault or hang.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nccl.h>
#include <signal.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "hkv.h"
#include "hkv_seqsplit.hpp"

extern "C" {
void hkv_oracle_fill(uint16_t* dst, uint64_t seed, uint64_t first_index, uint64_t count);
void hkv_oracle_append(const uint16_t* new_k, const uint16_t* new_v, uint16_t* k_cache, uint16_t* v_cache,
                       int B, int S, int KVH, int HD, int slots, int64_t batch_stride, const int32_t* pos,
                       int layout);
void hkv_oracle_decode(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out,
                       float* out_f32, int B, const int32_t* total, int H, int KVH, int HD, int slots,
                       int64_t batch_stride, float scale, int window, int layout, int mode, int threads);
float hkv_oracle_h2f(uint16_t h);
}

using namespace std::chrono_literals;

static int g_failures = 0;
#define REQUIRE(cond, msg)                                              \
    do {                                                                \
        if (!(cond)) {                                                  \
            std::printf("FAIL: %s (%s:%d)\n", msg, __FILE__, __LINE__); \
            ++g_failures;                                               \
        }                                                               \
    } while (0)
#define CUDA_OK(x)                                                                              \
    do {                                                                                        \
        const cudaError_t e_ = (x);                                                             \
        if (e_ != cudaSuccess) { std::printf("FAIL: %s: %s\n", #x, cudaGetErrorString(e_)); return 1; } \
    } while (0)

namespace {

constexpr int L = 3, B = 3, H = 28, KVH = 4, HD = 128, CTX = 2048, BLK = 128, STEPS = 6;

bool close_enough(const std::vector<uint16_t>& got, const std::vector<uint16_t>& ref, float* worst) {
    bool ok = true;
    for (size_t i = 0; i < got.size(); ++i) {
        const float g = hkv_oracle_h2f(got[i]), r = hkv_oracle_h2f(ref[i]);
        const float err = std::fabs(g - r);
        if (err > *worst) *worst = err;
        if (!(err <= 2e-3f + 1e-2f * std::fabs(r))) ok = false;   // the path's tolerance
    }
    return ok;
}

// Progress lines of a rank (unbuffered, so they survive a rank that is stopped at its time limit).
#define STAGE(...)                                       \
    do {                                                 \
        std::printf("[rank %d] ", rank);                 \
        std::printf(__VA_ARGS__);                        \
        std::printf("\n");                               \
    } while (0)

int run_rank(int rank, int world, const std::string& idfile, bool leave_at_end, const std::string& exchange) {
    setvbuf(stdout, nullptr, _IONBF, 0);
    CUDA_OK(cudaSetDevice(world > 1 ? rank : 0));
    ncclUniqueId id;
    std::memset(&id, 0, sizeof id);
    // Roster of the node's ranks (host-side presence board). Rank 0 creates it BEFORE it publishes
    // the communicator id; the others open it only after they have read the id.
    std::unique_ptr<hkv::NodeRoster> roster;
    const std::string rname = "/hkv-seqsplit-" + std::to_string((unsigned long)std::hash<std::string>{}(idfile));
    if (world > 1) {
        if (rank == 0) {
            roster.reset(new hkv::NodeRoster(rname, world, rank, true));
            if (ncclGetUniqueId(&id) != ncclSuccess) { std::printf("FAIL: ncclGetUniqueId\n"); return 1; }
            std::ofstream(idfile + ".tmp", std::ios::binary).write(reinterpret_cast<const char*>(&id), sizeof id);
            std::rename((idfile + ".tmp").c_str(), idfile.c_str());
        } else {
            const auto deadline = std::chrono::steady_clock::now() + 60s;
            for (;;) {
                std::ifstream f(idfile, std::ios::binary);
                if (f && f.read(reinterpret_cast<char*>(&id), sizeof id)) break;
                if (std::chrono::steady_clock::now() > deadline) { std::printf("FAIL: no communicator id\n"); return 1; }
                std::this_thread::sleep_for(20ms);
            }
            roster.reset(new hkv::NodeRoster(rname, world, rank));
        }
    }
    if (world > 1) STAGE("communicator id exchanged");
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));

    // Logical data, identical on every rank (seeded): planes [L][B][CTX][KVH][HD], per-step q/k_new/v_new.
    const size_t row = (size_t)KVH * HD, plane = (size_t)B * CTX * row, qn = (size_t)B * H * HD, kn = (size_t)B * row;
    std::vector<uint16_t> lk(L * plane), lv(L * plane);
    hkv_oracle_fill(lk.data(), 0x5153ull, 0, lk.size());
    hkv_oracle_fill(lv.data(), 0x5154ull, 0, lv.size());
    int32_t totals[B] = {1500, 700, 65};   // attended lengths AFTER the first append

    // This rank's share: logical block j lives on rank j % world as local block j / world.
    const int blocks = CTX / BLK, local_slots = ((blocks + world - 1) / world) * BLK;
    const size_t lplane = (size_t)B * local_slots * row;
    std::vector<uint16_t> sk(L * lplane, 0), sv(L * lplane, 0);
    auto local_row = [&](int p) { const int blk = p / BLK; return blk % world == rank ? (blk / world) * BLK + p % BLK : -1; };
    for (int l = 0; l < L; ++l)
        for (int b = 0; b < B; ++b)
            for (int p = 0; p < totals[b] - 1; ++p) {   // rows before the first new token
                const int r = local_row(p);
                if (r < 0) continue;
                std::memcpy(&sk[l * lplane + ((size_t)b * local_slots + r) * row], &lk[l * plane + ((size_t)b * CTX + p) * row], row * 2);
                std::memcpy(&sv[l * lplane + ((size_t)b * local_slots + r) * row], &lv[l * plane + ((size_t)b * CTX + p) * row], row * 2);
            }
    half *dk, *dv, *dq, *dkn, *dvn, *dout;
    int32_t* dtot;
    CUDA_OK(cudaMalloc(&dk, sk.size() * 2)); CUDA_OK(cudaMalloc(&dv, sv.size() * 2));
    CUDA_OK(cudaMalloc(&dq, L * qn * 2)); CUDA_OK(cudaMalloc(&dkn, L * kn * 2)); CUDA_OK(cudaMalloc(&dvn, L * kn * 2));
    CUDA_OK(cudaMalloc(&dout, L * qn * 2)); CUDA_OK(cudaMalloc(&dtot, sizeof totals));
    CUDA_OK(cudaMemcpy(dk, sk.data(), sk.size() * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dv, sv.data(), sv.size() * 2, cudaMemcpyHostToDevice));

    int rc = 0;
    try {
        hkv::SeqSplitConfig cfg;
        cfg.layers = L; cfg.batch = B; cfg.heads = H; cfg.kv_heads = KVH; cfg.head_dim = HD;
        cfg.local_slots = (uint32_t)local_slots; cfg.shard_block = BLK; cfg.rank = rank; cfg.world = world;
        cfg.exchange = exchange == "peer" ? hkv::Exchange::PeerStores : exchange == "nccl" ? hkv::Exchange::Nccl : hkv::Exchange::Auto;
        cfg.peer_wait_ms = 5000;
        hkv::SeqSplitDecoder dec(cfg, world > 1 ? &id : nullptr, stream);
        if (world > 1) STAGE("decoder and communicator ready (%s)", dec.exchange() == hkv::Exchange::PeerStores ? "mailboxes" : "all-gather");
        if (world > 1 && exchange == "peer") REQUIRE(dec.exchange() == hkv::Exchange::PeerStores, "mailboxes mapped on every rank");
        if (world == 1 || exchange == "nccl") REQUIRE(dec.exchange() == hkv::Exchange::Nccl, "no mailboxes unless asked for");
        dec.bind(dq, dkn, dvn, dout, dk, dv, lplane, dtot);
        if (roster) dec.attach_roster(roster.get(), 20000ms);

        std::vector<uint16_t> q(L * qn), nk(L * kn), nv(L * kn), got(L * qn), ref(qn);
        float worst = 0.0f;
        uint64_t replays = 0;
        for (int s = 0; s < STEPS; ++s) {
            hkv_oracle_fill(q.data(), 0x7100ull + s, 0, q.size());
            hkv_oracle_fill(nk.data(), 0x7200ull + s, 0, nk.size());
            hkv_oracle_fill(nv.data(), 0x7300ull + s, 0, nv.size());
            CUDA_OK(cudaMemcpyAsync(dq, q.data(), q.size() * 2, cudaMemcpyHostToDevice, stream));
            CUDA_OK(cudaMemcpyAsync(dkn, nk.data(), nk.size() * 2, cudaMemcpyHostToDevice, stream));
            CUDA_OK(cudaMemcpyAsync(dvn, nv.data(), nv.size() * 2, cudaMemcpyHostToDevice, stream));
            CUDA_OK(cudaMemcpyAsync(dtot, totals, sizeof totals, cudaMemcpyHostToDevice, stream));
            replays += dec.step() ? 1 : 0;
            const hkv::WatchResult w = dec.wait(30000ms);
            if (world > 1) STAGE("step %d %s (%s)", s, hkv::watch_result_name(w), dec.graph().valid() ? "graph" : "direct");
            REQUIRE(w == hkv::WatchResult::Done, "the step completes within its deadline");
            if (w != hkv::WatchResult::Done) throw std::runtime_error("step did not complete");
            CUDA_OK(cudaMemcpy(got.data(), dout, got.size() * 2, cudaMemcpyDeviceToHost));
            // host mirror: append at position total - 1 of the logical planes, attend
            int32_t pos[B];
            for (int b = 0; b < B; ++b) pos[b] = totals[b] - 1;
            for (int l = 0; l < L; ++l) {
                hkv_oracle_append(&nk[l * kn], &nv[l * kn], &lk[l * plane], &lv[l * plane], B, 1, KVH, HD, CTX,
                                  (int64_t)CTX * row, pos, 0);
                hkv_oracle_decode(&q[l * qn], &lk[l * plane], &lv[l * plane], ref.data(), nullptr, B, totals, H, KVH, HD, CTX,
                                  (int64_t)CTX * row, 1.0f / std::sqrt((float)HD), 0, 0, 0, 4);
                std::vector<uint16_t> g(got.begin() + l * qn, got.begin() + (l + 1) * qn);
                REQUIRE(close_enough(g, ref, &worst), "every rank's replicated output equals the oracle's");
            }
            for (int b = 0; b < B; ++b) ++totals[b];
        }
        REQUIRE(replays == STEPS - 1, "the first step runs un-captured; the second captures the graph and launches it; the rest replay");
        REQUIRE(dec.device_status() == 0, "device status word clean");
        // planes: this rank holds exactly its share of the logical planes, appended rows included
        CUDA_OK(cudaMemcpy(sk.data(), dk, sk.size() * 2, cudaMemcpyDeviceToHost));
        CUDA_OK(cudaMemcpy(sv.data(), dv, sv.size() * 2, cudaMemcpyDeviceToHost));
        bool planes_ok = true;
        for (int l = 0; l < L && planes_ok; ++l)
            for (int b = 0; b < B && planes_ok; ++b)
                for (int p = 0; p < totals[b] - 1; ++p) {
                    const int r = local_row(p);
                    if (r < 0) continue;
                    if (std::memcmp(&sk[l * lplane + ((size_t)b * local_slots + r) * row], &lk[l * plane + ((size_t)b * CTX + p) * row], row * 2) ||
                        std::memcmp(&sv[l * lplane + ((size_t)b * local_slots + r) * row], &lv[l * plane + ((size_t)b * CTX + p) * row], row * 2)) {
                        planes_ok = false;
                        break;
                    }
                }
        REQUIRE(planes_ok, "owner planes bit-exact (appended rows stored by their owner only)");
        std::printf("rank %d/%d (%s): %d steps, %llu replays, graph of %zu nodes, max abs err %.3e\n", rank, world,
                    dec.exchange() == hkv::Exchange::PeerStores ? "mailboxes" : "all-gather", STEPS,
                    (unsigned long long)replays, dec.graph().node_count(), worst);

        if (leave_at_end && world > 1) {
            // Between steps, nothing in flight (wait() returned Done on every rank's own stream).
            if (rank == world - 1) {
                roster->leave();
                std::printf("rank %d: left between steps\n", rank);
            } else {
                bool refused = false;
                std::string what;
                const auto deadline = std::chrono::steady_clock::now() + 20s;
                while (!refused && std::chrono::steady_clock::now() < deadline) {
                    if (!roster->has_left(world - 1)) { std::this_thread::sleep_for(5ms); continue; }
                    try { dec.step(); } catch (const std::exception& e) { refused = true; what = e.what(); }
                    break;
                }
                REQUIRE(refused, "the step after a peer's departure is refused on the host, before any launch");
                REQUIRE(what.find("has left") != std::string::npos, "and the message names the departure");
                REQUIRE(cudaStreamQuery(stream) == cudaSuccess, "nothing was enqueued");
            }
            dec.abandon();   // peers are no longer in step: tear the communicator down without them
        }
    } catch (const std::exception& e) {
        std::printf("FAIL: exception: %s\n", e.what());
        rc = 1;
    }
    cudaFree(dk); cudaFree(dv); cudaFree(dq); cudaFree(dkn); cudaFree(dvn); cudaFree(dout); cudaFree(dtot);
    cudaStreamDestroy(stream);
    if (roster && rank == 0) roster->unlink();
    if (g_failures) rc = 1;
    std::printf("%s: rank %d\n", rc ? "FAIL" : "PASS", rank);
    return rc;
}

}  // namespace

int main(int argc, char** argv) {
    int rank = -1, world = 0;
    std::string idfile;
    bool leave = false;
    std::string exchange = "auto";
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--list") { std::printf("seqsplit_decoder\n"); return 0; }
        if (a == "--rank" && i + 1 < argc) rank = std::atoi(argv[++i]);
        else if (a == "--world" && i + 1 < argc) world = std::atoi(argv[++i]);
        else if (a == "--idfile" && i + 1 < argc) idfile = argv[++i];
        else if (a == "--exchange" && i + 1 < argc) exchange = argv[++i];
        else if (a == "--leave") leave = true;
    }
    if (rank >= 0) return run_rank(rank, world, idfile, leave, exchange);

    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("FAIL: no CUDA device\n"); return 1; }
    if (world <= 0) world = ndev < 4 ? ndev : 4;
    if (world > ndev) { std::printf("FAIL: %d ranks asked, %d GPUs present\n", world, ndev); return 1; }
    if (world == 1) {
        const int rc = run_rank(0, 1, "", false, "auto");
        if (!rc) std::printf("ALL PASSED (world 1)\n");
        return rc;
    }
    // one child per GPU, each this binary with --rank; the whole sequence once per exchange
    setenv("NCCL_NVLS_ENABLE", "0", 0);   // a rank leaves at the end of this test: keep multicast objects out of it
    int bad = 0;
    for (const char* mode : {"nccl", "peer"}) {
        char tmpl[] = "/tmp/hkv-seqsplit-id-XXXXXX";
        const int fd = mkstemp(tmpl);
        if (fd >= 0) { close(fd); unlink(tmpl); }
        idfile = tmpl;
        std::printf("== exchange: %s\n", mode);
        std::vector<pid_t> kids;
        for (int r = 0; r < world; ++r) {
            const pid_t pid = fork();
            if (pid == 0) {
                const std::string rs = std::to_string(r), ws = std::to_string(world);
                execl(argv[0], argv[0], "--rank", rs.c_str(), "--world", ws.c_str(), "--idfile", idfile.c_str(), "--exchange", mode,
                      "--leave", (char*)nullptr);
                _exit(127);
            }
            kids.push_back(pid);
        }
        const auto deadline = std::chrono::steady_clock::now() + 150s;
        std::vector<bool> done(kids.size(), false);
        size_t left = kids.size();
        while (left && std::chrono::steady_clock::now() < deadline) {
            for (size_t i = 0; i < kids.size(); ++i) {
                if (done[i]) continue;
                int status = 0;
                if (waitpid(kids[i], &status, WNOHANG) == kids[i]) {
                    done[i] = true;
                    --left;
                    if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) ++bad;
                }
            }
            std::this_thread::sleep_for(50ms);
        }
        for (size_t i = 0; i < kids.size(); ++i)
            if (!done[i]) { kill(kids[i], SIGKILL); waitpid(kids[i], nullptr, 0); ++bad; std::printf("FAIL: rank %zu exceeded the time limit\n", i); }
        unlink(idfile.c_str());
        if (bad) break;
    }
    if (!bad) std::printf("ALL PASSED (world %d)\n", world);
    return bad ? 1 : 0;
}
