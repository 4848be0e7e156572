// The barrier between the ranks of a communicator, as one step that both the device kernel
// and a host-side test instantiate: the caller says "rank `rank` has reached generation
// `epoch`" to every peer (a store into the peer's flag array) and then waits, at most
// max_polls polls per peer, until every peer has said the same here.  Returns false when a
// wait ran out.  Generations compare modulo 2^32.  `Memory` supplies the release store, the
// acquire load and the pause between polls for the address space at hand.
#pragma once

#if defined(__CUDACC__)
#define B200ALG_HD __host__ __device__
#else
#define B200ALG_HD
#endif

namespace b200alg {

template <typename Memory>
B200ALG_HD inline void rank_barrier_signal(Memory &mem, unsigned int *peer_flags_of_b, int rank, unsigned int epoch) {
    mem.store_release(peer_flags_of_b + rank, epoch);
}

template <typename Memory>
B200ALG_HD inline bool rank_barrier_wait(Memory &mem, const unsigned int *my_flags, int peer, unsigned int epoch,
                                         unsigned int max_polls) {
    unsigned int polls = 0;
    while ((int)(mem.load_acquire(my_flags + peer) - epoch) < 0) {
        if (++polls > max_polls) return false;
        mem.pause();
    }
    return true;
}

}  // namespace b200alg
