// The rank barrier of the multi-GPU library (ilgpu_b200/csrc/rank_barrier.cuh) on the host: two
// threads stand for two ranks, std::atomic for the mapped flag arrays.  Case 1: both ranks arrive,
// several generations in a row.  Case 2: one rank never arrives; the other gives up after its
// poll limit and reports it instead of hanging.  No GPU involved.
#include <atomic>
#include <cstdio>
#include <thread>

#include "rank_barrier.cuh"

struct HostMemory {
    void store_release(unsigned int *p, unsigned int v) { reinterpret_cast<std::atomic<unsigned int> *>(p)->store(v, std::memory_order_release); }
    unsigned int load_acquire(const unsigned int *p) { return reinterpret_cast<const std::atomic<unsigned int> *>(p)->load(std::memory_order_acquire); }
    void pause() { std::this_thread::yield(); }
};

static int g_checks = 0, g_failures = 0;
#define CHECK(cond)                                                             \
    do {                                                                        \
        ++g_checks;                                                             \
        if (!(cond)) { ++g_failures; std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)

int main() {
    alignas(64) static unsigned int flags[2][2] = {{0, 0}, {0, 0}};   // flags[r][b]: what rank b told rank r
    unsigned int *peer_flags[2] = {flags[0], flags[1]};

    // 1. both ranks take part, 1000 generations; a payload written before the barrier is visible after it
    static int payload[2] = {0, 0};
    bool ok[2] = {true, true};
    auto rank_main = [&](int rank) {
        HostMemory mem;
        for (unsigned int round = 1; round <= 1000; ++round) {
            payload[rank] = (int)round;
            const unsigned int first = 2 * round - 1, second = 2 * round;   // generations only ever grow
            for (int b = 0; b < 2; ++b) b200alg::rank_barrier_signal(mem, peer_flags[b], rank, first);
            for (int b = 0; b < 2; ++b) ok[rank] = ok[rank] && b200alg::rank_barrier_wait(mem, flags[rank], b, first, 1u << 30);
            ok[rank] = ok[rank] && payload[1 - rank] == (int)round;
            // a second barrier keeps the other rank from racing ahead into the next payload write
            for (int b = 0; b < 2; ++b) b200alg::rank_barrier_signal(mem, peer_flags[b], rank, second);
            for (int b = 0; b < 2; ++b) ok[rank] = ok[rank] && b200alg::rank_barrier_wait(mem, flags[rank], b, second, 1u << 30);
        }
    };
    {
        std::thread t0(rank_main, 0), t1(rank_main, 1);
        t0.join();
        t1.join();
    }
    CHECK(ok[0] && ok[1]);

    // 2. rank 1 never arrives: rank 0's wait for it runs out after 1000 polls and says so
    {
        HostMemory mem;
        const unsigned int epoch = 500000;   // later than every generation of case 1
        for (int b = 0; b < 2; ++b) b200alg::rank_barrier_signal(mem, peer_flags[b], 0, epoch);
        CHECK(b200alg::rank_barrier_wait(mem, flags[0], 0, epoch, 1000));     // its own flag is there
        CHECK(!b200alg::rank_barrier_wait(mem, flags[0], 1, epoch, 1000));    // the absent rank's is not
    }
    // 3. generations compare modulo 2^32: a flag just past the wrap counts as "later"
    {
        HostMemory mem;
        mem.store_release(&flags[0][1], 3u);
        CHECK(b200alg::rank_barrier_wait(mem, flags[0], 1, 0xFFFFFFF0u, 10));
    }
    std::printf("rank barrier on the host: %d checks, %d failures\n", g_checks, g_failures);
    return g_failures ? 1 : 0;
}
