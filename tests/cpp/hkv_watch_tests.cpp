// hkv_watch_tests.cpp — CPU-only tests of the host-side failure detection of the multi-GPU step
// (host/hkv_step_watch.hpp). No CUDA, no GPU: the failures are made on the host — a collective
// that never completes, a communicator that reports an error, a rank that leaves between steps or
// never joins — with threads and forked processes standing in for the ranks.
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <string>
#include <thread>
#include <vector>

#include "hkv_step_watch.hpp"

using namespace std::chrono_literals;
using hkv::NodeRoster;
using hkv::WatchResult;

static int g_failures = 0;
#define REQUIRE(cond, msg)                                              \
    do {                                                                \
        if (!(cond)) {                                                  \
            std::printf("FAIL: %s (%s:%d)\n", msg, __FILE__, __LINE__); \
            ++g_failures;                                               \
        }                                                               \
    } while (0)

static std::string roster_name(const char* tag) { return std::string("/hkv-test-") + tag + "-" + std::to_string(getpid()); }

// A step that completes, one whose communicator fails, one that never completes.
static void test_watch_step() {
    int polls = 0;
    WatchResult r = hkv::watch_step([&] { return ++polls >= 5; }, [] { return false; }, 2000ms, 0us);
    REQUIRE(r == WatchResult::Done && polls == 5, "a step that completes is Done");

    polls = 0;
    r = hkv::watch_step([] { return false; }, [&] { return ++polls >= 3; }, 2000ms, 0us);
    REQUIRE(r == WatchResult::PeerError && polls == 3, "an asynchronous communicator error ends the wait");

    // error and completion in the same poll: the error wins (a failed collective may look complete)
    r = hkv::watch_step([] { return true; }, [] { return true; }, 2000ms, 0us);
    REQUIRE(r == WatchResult::PeerError, "the error check comes first");

    const auto t0 = std::chrono::steady_clock::now();
    r = hkv::watch_step([] { return false; }, [] { return false; }, 50ms);
    const auto dt = std::chrono::steady_clock::now() - t0;
    REQUIRE(r == WatchResult::TimedOut, "a step that never completes times out");
    REQUIRE(dt >= 50ms && dt < 1000ms, "the wait honours its deadline");
}

// Four thread-ranks step together; rank 2 leaves after step 3: every other rank must refuse step 4
// BEFORE launching it, naming rank 2.
static void test_roster_rank_leaves_between_steps() {
    const std::string name = roster_name("leave");
    const int world = 4;
    { NodeRoster init(name, world, 0, /*fresh=*/true); }
    std::atomic<int> barrier_count{0};
    std::atomic<bool> gone{false};   // test choreography only: step 4 starts after rank 2 is gone
    std::vector<int> refused_at(world, 0), offender(world, -1);
    auto rank_main = [&](int rank) {
        NodeRoster roster(name, world, rank);
        for (uint64_t step = 1; step <= 6; ++step) {
            if (rank == 2 && step == 4) { roster.leave(); gone.store(true); return; }
            if (step == 4) while (!gone.load()) std::this_thread::yield();
            roster.announce(step);
            int who = -1;
            const NodeRoster::Check c = roster.check_before_launch(step, 2000ms, &who);
            if (c != NodeRoster::Check::Ok) { refused_at[rank] = (int)step; offender[rank] = who; return; }
            // the "collective" of the step: everybody meets
            const int target = (int)step * world - (step > 3 ? (int)(step - 3) : 0);
            barrier_count.fetch_add(1);
            const auto deadline = std::chrono::steady_clock::now() + 2000ms;
            while (barrier_count.load() < target && std::chrono::steady_clock::now() < deadline) std::this_thread::yield();
        }
    };
    std::vector<std::thread> ts;
    for (int r = 0; r < world; ++r) ts.emplace_back(rank_main, r);
    for (auto& t : ts) t.join();
    for (int r = 0; r < world; ++r) {
        if (r == 2) continue;
        REQUIRE(refused_at[r] == 4, "every remaining rank refuses the step after the departure");
        REQUIRE(offender[r] == 2, "and names the rank that left");
    }
    NodeRoster(name, world, 0).unlink();
}

// A rank that never joins (its process died at start-up): the others give up after the grace period.
static void test_roster_rank_never_joins() {
    const std::string name = roster_name("nojoin");
    NodeRoster r0(name, 3, 0, true);
    NodeRoster r1(name, 3, 1);
    r0.announce(1);
    r1.announce(1);
    int who = -1;
    const auto t0 = std::chrono::steady_clock::now();
    const NodeRoster::Check c = r0.check_before_launch(1, 100ms, &who);
    const auto dt = std::chrono::steady_clock::now() - t0;
    REQUIRE(c == NodeRoster::Check::PeerBehind && who == 2, "a rank that never joined is reported as behind");
    REQUIRE(dt >= 100ms && dt < 2000ms, "after the grace period, not before");
    r0.unlink();
}

// Real processes: the roster lives in POSIX shared memory. The child steps twice and exits after
// announcing its departure; the parent sees steps, then the departure.
static void test_roster_across_processes() {
    const std::string name = roster_name("fork");
    NodeRoster parent(name, 2, 0, true);
    const pid_t pid = fork();
    if (pid == 0) {
        NodeRoster child(name, 2, 1);
        child.announce(1);
        std::this_thread::sleep_for(50ms);
        child.announce(2);
        std::this_thread::sleep_for(50ms);
        child.leave();
        _exit(0);
    }
    parent.announce(1);
    REQUIRE(parent.check_before_launch(1, 2000ms) == NodeRoster::Check::Ok, "step 1: the child process is present");
    parent.announce(2);
    REQUIRE(parent.check_before_launch(2, 2000ms) == NodeRoster::Check::Ok, "step 2: still present");
    int status = 0;
    waitpid(pid, &status, 0);
    parent.announce(3);
    int who = -1;
    REQUIRE(parent.check_before_launch(3, 2000ms, &who) == NodeRoster::Check::PeerLeft && who == 1,
            "step 3: the departure of the child process is seen before the launch");
    parent.unlink();
}

// A straggler one step behind is fine (ranks run at most a step apart); two steps behind is not.
static void test_roster_straggler() {
    const std::string name = roster_name("lag");
    NodeRoster a(name, 2, 0, true), b(name, 2, 1);
    b.announce(4);
    a.announce(5);
    REQUIRE(a.check_before_launch(5, 50ms) == NodeRoster::Check::Ok, "a peer one step behind will still join");
    a.announce(6);
    int who = -1;
    REQUIRE(a.check_before_launch(6, 50ms, &who) == NodeRoster::Check::PeerBehind && who == 1, "two steps behind is reported");
    bool threw = false;
    try { NodeRoster bad(name, 2, 2); } catch (const std::exception&) { threw = true; }
    REQUIRE(threw, "a rank outside the world is refused");
    a.unlink();
}

int main(int argc, char** argv) {
    struct Case { const char* name; void (*fn)(); };
    const Case cases[] = {{"watch_step", test_watch_step},
                          {"roster_rank_leaves_between_steps", test_roster_rank_leaves_between_steps},
                          {"roster_rank_never_joins", test_roster_rank_never_joins},
                          {"roster_across_processes", test_roster_across_processes},
                          {"roster_straggler", test_roster_straggler}};
    if (argc > 1 && std::string(argv[1]) == "--list") {
        for (const Case& c : cases) std::printf("%s\n", c.name);
        return 0;
    }
    for (const Case& c : cases) {
        const int before = g_failures;
        c.fn();
        std::printf("%s: %s\n", g_failures == before ? "PASS" : "FAIL", c.name);
    }
    if (g_failures == 0) std::printf("ALL PASSED\n");
    return g_failures ? 1 : 0;
}
