// The primitives over the GPUs of one box: one communicator per GPU, NCCL for the few words
// every primitive has to exchange, peer stores for the buckets of the sort.
// New surface (the reference has no multi-device algorithms; Src/ILGPU/Runtime/PeerAccess.cs
// is its only multi-GPU facility).  Built into libb200alg_mg.so, which uses the single-GPU
// entry points of libb200alg.so for all local work.
#include <nccl.h>
#include <pthread.h>
#include <unistd.h>

#include <cstring>
#include <type_traits>
#include <utility>
#include <vector>

#include "common.cuh"
#include "rank_barrier.cuh"
#include "../../include/b200alg_mg.h"

namespace b200alg {

constexpr int kMaxRanks = 16;
constexpr int kSamplesPerRank = 2048;
// The flag allocation of a rank is mapped into every other rank.  Behind the barrier flags it
// holds two mailboxes that the others store into directly (peer stores over NVLink, made
// visible by the barrier that follows): the sample messages and the rows of the bucket-size
// matrix of the sort in flight.
constexpr int64_t kFlagBytes = 256;
constexpr int64_t kSampleMessageWords = 2 * kSamplesPerRank + 1;
constexpr int64_t kSampleMailboxAt = kFlagBytes;
constexpr int64_t kMatrixMailboxAt = kSampleMailboxAt + 8ll * kMaxRanks * kSampleMessageWords;
constexpr int64_t kMailboxEnd = kMatrixMailboxAt + 8ll * kMaxRanks * (kMaxRanks + 1);
// Position of element i of rank r in the tie-breaking order of the sort: r * 2^40 + i.  It only
// has to be monotone in (rank, position).
constexpr int kRankShift = 40;
// Polls of a flag another GPU sets before a barrier gives up (about a second).
constexpr unsigned int kMaxFlagPolls = 1u << 21;

// What a rank tells the others about its memory when the communicator is built.
struct PeerInfo {
    long long pid;
    unsigned long long host_hash;
    unsigned long long recv_ptr, flag_ptr;       // raw device addresses (meaningful inside the owner's process)
    cudaIpcMemHandle_t recv_handle, flag_handle; // for other processes
    int device;
    int pad;
};

// Device-resident words of a communicator.
struct CommState {
    TempHeader hdr;                    // hdr.wait_limit_hit: a bounded wait ran out / receive buffer too small
    long long recv_count;              // elements this rank received in the current sort
    long long bucket_counts[kMaxRanks + 1];              // sizes of this shard's buckets
    void *key_ptrs[kMaxRanks];         // where bucket b of this rank's shard goes
    void *value_ptrs[kMaxRanks];
    long long sample_count;            // valid samples of the current sort
    unsigned long long splitter_keys[kMaxRanks];  // raw key bits, element size of the key type
    long long splitter_index[kMaxRanks];
    unsigned long long scalar[4];      // reduce / scan totals in flight
    unsigned long long gathered[kMaxRanks * 2];
};

}  // namespace b200alg

struct b200alg_comm {
    ncclComm_t nccl = nullptr;
    int rank = 0, ranks = 1, device = 0;
    int last_nccl = 0;
    int64_t capacity = 0;           // elements per receive buffer
    unsigned int epoch = 0;         // barrier generation
    b200alg::CommState *state = nullptr;    // device
    unsigned char *recv = nullptr;          // device: keys at 0, values at capacity * 8
    unsigned int *flags = nullptr;          // device: flags[r] = last barrier generation rank r reached
    void *peer_recv[b200alg::kMaxRanks] = {};   // this rank's view of every rank's receive buffer
    unsigned int *peer_flags[b200alg::kMaxRanks] = {};
    bool opened_recv[b200alg::kMaxRanks] = {}, opened_flags[b200alg::kMaxRanks] = {};
    void **d_peer_recv = nullptr;           // device copies of the two tables
    unsigned int **d_peer_flags = nullptr;
    unsigned char *scratch = nullptr;       // device: sample arrays, partition temp, sort temp, histogram bins
    int64_t off_sample_keys = 0, off_sample_index = 0,
            off_partition_temp = 0, partition_temp_bytes = 0, off_sort_temp = 0, sort_temp_bytes = 0,
            off_sink = 0, off_bins = 0, scratch_bytes = 0;
};

namespace b200alg {

#define B200ALG_NCCL_TRY(comm, expr)                   \
    do {                                               \
        ncclResult_t _r = (expr);                      \
        if (_r != ncclSuccess) {                       \
            (comm)->last_nccl = (int)_r;               \
            return B200ALG_NCCL_ERROR;                 \
        }                                              \
    } while (0)

static bool nccl_type(int dtype, ncclDataType_t *t) {
    switch (dtype) {
    case B200ALG_I32: *t = ncclInt32; return true;
    case B200ALG_U32: *t = ncclUint32; return true;
    case B200ALG_I64: *t = ncclInt64; return true;
    case B200ALG_U64: *t = ncclUint64; return true;
    case B200ALG_F32: *t = ncclFloat32; return true;
    case B200ALG_F64: *t = ncclFloat64; return true;
    }
    return false;
}
static ncclRedOp_t nccl_op(int op) { return op == B200ALG_ADD ? ncclSum : (op == B200ALG_MAX ? ncclMax : ncclMin); }

__device__ __forceinline__ void st_release_sys_u32(unsigned int *p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Barrier over the ranks, on the stream: thread b tells rank b that this rank has reached
// generation `epoch` (a store into rank b's flag array, which is mapped here) and waits until
// rank b has said the same here (rank_barrier.cuh).  The wait is bounded; when it runs out the
// kernel records that and returns.
struct SystemScopeMemory {
    __device__ void store_release(unsigned int *p, unsigned int v) { st_release_sys_u32(p, v); }
    __device__ unsigned int load_acquire(const unsigned int *p) { return ld_acquire_sys_u32(p); }
    __device__ void pause() { __nanosleep(200); }
};
__global__ void rank_barrier_kernel(unsigned int *const *peer_flags, const unsigned int *my_flags, int rank, int ranks,
                                    unsigned int epoch, TempHeader *hdr) {
    const int b = threadIdx.x;
    if (b >= ranks) return;
    SystemScopeMemory mem;
    __threadfence_system();  // everything this GPU wrote before (peer stores of the kernel before) goes first
    rank_barrier_signal(mem, peer_flags[b], rank, epoch);
    if (!rank_barrier_wait(mem, my_flags, b, epoch, kMaxFlagPolls)) atomicExch(&hdr->wait_limit_hit, 1u);
}

// ---- reduce / scan helpers -----------------------------------------------------------------
// Rank-ordered fold of the totals of the ranks below `rank` (floating-point sums in double).
template <typename T, int OP>
__global__ void fold_lower_kernel(const T *totals, int rank, T *carry) {
    using O = Op<T, OP>;
    if (threadIdx.x != 0) return;
    if (OP == B200ALG_ADD && std::is_same<T, float>::value) {
        double acc = 0.0;
        for (int r = 0; r < rank; ++r) acc += (double)totals[r];
        *carry = (T)acc;
    } else {
        T acc = O::identity();
        for (int r = 0; r < rank; ++r) acc = O::apply(acc, totals[r]);
        *carry = acc;
    }
}

template <typename T> __global__ void set_identity_kernel(T *cell, T v) { *cell = v; }

// ---- histogram helpers -----------------------------------------------------------------------
// bins += summed counts of all ranks; overflow as the single-GPU kernel decides it for one
// block's count (the reference raises the flag when a single increment starts from MaxValue).
__global__ void add_bins_kernel(void *bins, const void *counts, int64_t num_bins, int bin_dtype, int *overflow) {
    bool of = false;
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < num_bins; b += (int64_t)gridDim.x * blockDim.x) {
        switch (bin_dtype) {
        case B200ALG_I32: case B200ALG_U32: {
            const unsigned int c = ((const unsigned int *)counts)[b];
            const unsigned int old = ((unsigned int *)bins)[b];
            ((unsigned int *)bins)[b] = old + c;
            const unsigned int top = bin_dtype == B200ALG_I32 ? 0x7FFFFFFFu : 0xFFFFFFFFu;
            of |= (unsigned int)(top - old) < c;
            break;
        }
        case B200ALG_I64: case B200ALG_U64: {
            const unsigned long long c = ((const unsigned long long *)counts)[b];
            const unsigned long long old = ((unsigned long long *)bins)[b];
            ((unsigned long long *)bins)[b] = old + c;
            const unsigned long long top = bin_dtype == B200ALG_I64 ? 0x7FFFFFFFFFFFFFFFull : 0xFFFFFFFFFFFFFFFFull;
            of |= (top - old) < c;
            break;
        }
        case B200ALG_F32: {
            const float old = ((float *)bins)[b];
            ((float *)bins)[b] = old + ((const float *)counts)[b];
            of |= old == FLT_MAX && ((const float *)counts)[b] != 0.0f;
            break;
        }
        default: {
            const double old = ((double *)bins)[b];
            ((double *)bins)[b] = old + ((const double *)counts)[b];
            of |= old == DBL_MAX && ((const double *)counts)[b] != 0.0;
            break;
        }
        }
    }
    if (overflow && of) atomicOr(overflow, 1);
}

// ---- sort helpers --------------------------------------------------------------------------
// Message of one rank: [0] shard size, [1 .. 1+s) sampled keys (raw bits, zero-extended),
// [1+s .. 1+2s) their positions in the tie-breaking order.  Stored into slot `rank` of every
// rank's sample mailbox.
template <typename K>
__global__ void sample_kernel(const K *keys, int64_t n, int rank, int ranks, unsigned int *const *peer_flags) {
    const int s = kSamplesPerRank;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < s; i += gridDim.x * blockDim.x) {
        long long key = 0, pos = 0;
        if (n > 0) {
            const int64_t at = ((int64_t)i * n) / s;
            key = (long long)(unsigned long long)keys[at];
            pos = ((long long)rank << kRankShift) + at;
        }
        for (int r = 0; r < ranks; ++r) {
            long long *msg = reinterpret_cast<long long *>(reinterpret_cast<unsigned char *>(peer_flags[r]) + kSampleMailboxAt) +
                             (int64_t)rank * kSampleMessageWords;
            if (i == 0) msg[0] = n;
            msg[1 + i] = key;
            msg[1 + s + i] = pos;
        }
    }
}

// Row `rank` of the bucket-size matrix (this shard's bucket sizes, then this rank's output
// capacity) into every rank's matrix mailbox.
__global__ void publish_counts_kernel(const long long *bucket_counts, long long out_capacity, int rank, int ranks,
                                      unsigned int *const *peer_flags) {
    const int j = threadIdx.x;
    if (j > ranks) return;
    const long long v = j < ranks ? bucket_counts[j] : out_capacity;
    for (int r = 0; r < ranks; ++r) {
        long long *matrix = reinterpret_cast<long long *>(reinterpret_cast<unsigned char *>(peer_flags[r]) + kMatrixMailboxAt);
        matrix[rank * (ranks + 1) + j] = v;
    }
}

// Samples of the ranks that have data, in rank order, as a key array and an index array.
template <typename K>
__global__ void collect_samples_kernel(const long long *all, int ranks, K *sample_keys, long long *sample_index, long long *count) {
    const int s = kSamplesPerRank;
    const int stride_msg = 2 * s + 1;
    for (int r = blockIdx.x; r < ranks; r += gridDim.x) {
        const long long *msg = all + (int64_t)r * stride_msg;
        if (msg[0] <= 0) continue;
        int before = 0;
        for (int q = 0; q < r; ++q) before += all[(int64_t)q * stride_msg] > 0 ? 1 : 0;
        for (int i = threadIdx.x; i < s; i += blockDim.x) {
            sample_keys[(int64_t)before * s + i] = (K)(unsigned long long)msg[1 + i];
            sample_index[(int64_t)before * s + i] = msg[1 + s + i];
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        int with_data = 0;
        for (int q = 0; q < ranks; ++q) with_data += all[(int64_t)q * stride_msg] > 0 ? 1 : 0;
        *count = (long long)with_data * s;
    }
}

// From the matrix of bucket sizes (matrix[src][dst], the same on every rank): where this rank's
// buckets start inside the owners' receive buffers, how much this rank receives, and whether
// every receive buffer is large enough.  If one is not, every rank sends its buckets into a
// local sink instead, receives nothing and raises the flag.
__global__ void plan_exchange_kernel(CommState *st, const long long *matrix, void *const *peer_recv, int rank, int ranks,
                                     long long capacity, int key_bytes, int value_bytes, void *sink) {
    if (threadIdx.x != 0) return;
    const int row = ranks + 1;  // bucket sizes, then the source rank's output capacity
    bool fits = true;
    for (int b = 0; b < ranks; ++b) {
        long long column = 0;
        for (int src = 0; src < ranks; ++src) column += matrix[src * row + b];
        if (column > capacity || column > matrix[b * row + ranks]) fits = false;
    }
    long long mine = 0;
    for (int src = 0; src < ranks; ++src) mine += matrix[src * row + rank];
    for (int b = 0; b < ranks; ++b) {
        long long start = 0;
        for (int src = 0; src < rank; ++src) start += matrix[src * row + b];
        if (fits) {
            st->key_ptrs[b] = (unsigned char *)peer_recv[b] + start * key_bytes;
            st->value_ptrs[b] = (unsigned char *)peer_recv[b] + capacity * 8 + start * value_bytes;
        } else {
            st->key_ptrs[b] = sink;
            st->value_ptrs[b] = sink;
        }
    }
    st->recv_count = fits ? mine : 0;
    if (!fits) atomicExch(&st->hdr.wait_limit_hit, 1u);
}

static unsigned long long host_hash() {
    char name[256] = {0};
    gethostname(name, sizeof(name) - 1);
    unsigned long long h = 1469598103934665603ull;
    for (const char *p = name; *p; ++p) h = (h ^ (unsigned char)*p) * 1099511628211ull;
    return h;
}

// Allocations, the exchange of the memory handles and the peer mappings; the NCCL communicator
// exists already.  Collective.
static int finish_comm(b200alg_comm *c, int64_t sort_capacity, cudaStream_t s) {
    const int G = c->ranks;
    c->capacity = sort_capacity < 0 ? 0 : sort_capacity;
    B200ALG_CUDA_TRY(cudaMalloc((void **)&c->state, sizeof(CommState)));
    B200ALG_CUDA_TRY(cudaMemsetAsync(c->state, 0, sizeof(CommState), s));
    B200ALG_CUDA_TRY(cudaMalloc((void **)&c->flags, (size_t)kMailboxEnd));
    B200ALG_CUDA_TRY(cudaMemsetAsync(c->flags, 0, (size_t)kMailboxEnd, s));
    const int64_t recv_bytes = round_up(c->capacity * 16 + 256, 256);
    B200ALG_CUDA_TRY(cudaMalloc((void **)&c->recv, (size_t)recv_bytes));

    // scratch layout
    const int64_t total_samples = (int64_t)G * kSamplesPerRank;
    int64_t off = 0;
    auto take = [&](int64_t bytes) { const int64_t at = off; off += round_up(bytes, 256); return at; };
    c->off_sample_keys = take(total_samples * 8);
    c->off_sample_index = take(total_samples * 8);
    c->off_bins = take(1 << 20);  // local bin counts of the histogram (up to 128 Ki 8-byte bins)
    int64_t need = 0;
    const int64_t cap1 = c->capacity < 1 ? 1 : c->capacity;
    {
        int64_t a = 0;
        if (b200alg_radix_sort_temp_bytes(B200ALG_U64, cap1, 8, &a) != B200ALG_OK) return B200ALG_INVALID_ARGUMENT;
        const int64_t b = total_samples * 4;  // the ranks of the samples while the splitters are picked
        need = a > b ? a : b;
    }
    c->sort_temp_bytes = need;
    c->off_sort_temp = take(need);
    if (b200alg_bucket_partition_temp_bytes(B200ALG_U64, cap1, &need) != B200ALG_OK) return B200ALG_INVALID_ARGUMENT;
    c->partition_temp_bytes = need;
    c->off_partition_temp = take(need);
    c->off_sink = take(cap1 * 8);
    c->scratch_bytes = off;
    B200ALG_CUDA_TRY(cudaMalloc((void **)&c->scratch, (size_t)c->scratch_bytes));

    // tell the others where this rank's receive buffer and flags are
    PeerInfo mine;
    memset(&mine, 0, sizeof(mine));
    mine.pid = (long long)getpid();
    mine.host_hash = host_hash();
    mine.recv_ptr = (unsigned long long)(uintptr_t)c->recv;
    mine.flag_ptr = (unsigned long long)(uintptr_t)c->flags;
    mine.device = c->device;
    B200ALG_CUDA_TRY(cudaIpcGetMemHandle(&mine.recv_handle, c->recv));
    B200ALG_CUDA_TRY(cudaIpcGetMemHandle(&mine.flag_handle, c->flags));
    PeerInfo *d_info = nullptr;
    B200ALG_CUDA_TRY(cudaMalloc((void **)&d_info, sizeof(PeerInfo) * (G + 1)));
    B200ALG_CUDA_TRY(cudaMemcpyAsync(d_info + G, &mine, sizeof(mine), cudaMemcpyHostToDevice, s));
    B200ALG_NCCL_TRY(c, ncclAllGather(d_info + G, d_info, sizeof(PeerInfo), ncclChar, c->nccl, s));
    std::vector<PeerInfo> all(G);
    B200ALG_CUDA_TRY(cudaMemcpyAsync(all.data(), d_info, sizeof(PeerInfo) * G, cudaMemcpyDeviceToHost, s));
    B200ALG_CUDA_TRY(cudaStreamSynchronize(s));
    B200ALG_CUDA_TRY(cudaFree(d_info));
    for (int r = 0; r < G; ++r) {
        if (r == c->rank) {
            c->peer_recv[r] = c->recv;
            c->peer_flags[r] = c->flags;
        } else if (all[r].pid == mine.pid && all[r].host_hash == mine.host_hash) {
            // same process: the raw address is valid here once peer access is on
            int can = 0;
            B200ALG_CUDA_TRY(cudaDeviceCanAccessPeer(&can, c->device, all[r].device));
            if (!can) return B200ALG_UNSUPPORTED;
            const cudaError_t e = cudaDeviceEnablePeerAccess(all[r].device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return cuda_fail(e);
            (void)cudaGetLastError();
            c->peer_recv[r] = (void *)(uintptr_t)all[r].recv_ptr;
            c->peer_flags[r] = (unsigned int *)(uintptr_t)all[r].flag_ptr;
        } else {
            if (all[r].host_hash != mine.host_hash) return B200ALG_UNSUPPORTED;  // one box only
            B200ALG_CUDA_TRY(cudaIpcOpenMemHandle(&c->peer_recv[r], all[r].recv_handle, cudaIpcMemLazyEnablePeerAccess));
            c->opened_recv[r] = true;
            void *f = nullptr;
            B200ALG_CUDA_TRY(cudaIpcOpenMemHandle(&f, all[r].flag_handle, cudaIpcMemLazyEnablePeerAccess));
            c->peer_flags[r] = (unsigned int *)f;
            c->opened_flags[r] = true;
        }
    }
    B200ALG_CUDA_TRY(cudaMalloc((void **)&c->d_peer_recv, sizeof(void *) * kMaxRanks));
    B200ALG_CUDA_TRY(cudaMalloc((void **)&c->d_peer_flags, sizeof(void *) * kMaxRanks));
    B200ALG_CUDA_TRY(cudaMemcpyAsync(c->d_peer_recv, c->peer_recv, sizeof(void *) * kMaxRanks, cudaMemcpyHostToDevice, s));
    B200ALG_CUDA_TRY(cudaMemcpyAsync(c->d_peer_flags, c->peer_flags, sizeof(void *) * kMaxRanks, cudaMemcpyHostToDevice, s));
    B200ALG_CUDA_TRY(cudaStreamSynchronize(s));
    return B200ALG_OK;
}

static int rank_barrier(b200alg_comm *c, cudaStream_t s) {
    c->epoch += 1;
    rank_barrier_kernel<<<1, 32, 0, s>>>(c->d_peer_flags, c->flags, c->rank, c->ranks, c->epoch, &c->state->hdr);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

template <typename T>
static int fold_lower(cudaStream_t s, int op, const void *totals, int rank, void *carry) {
    switch (op) {
    case B200ALG_ADD: fold_lower_kernel<T, B200ALG_ADD><<<1, 32, 0, s>>>((const T *)totals, rank, (T *)carry); break;
    case B200ALG_MAX: fold_lower_kernel<T, B200ALG_MAX><<<1, 32, 0, s>>>((const T *)totals, rank, (T *)carry); break;
    case B200ALG_MIN: fold_lower_kernel<T, B200ALG_MIN><<<1, 32, 0, s>>>((const T *)totals, rank, (T *)carry); break;
    default: return B200ALG_UNSUPPORTED;
    }
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

template <typename T>
static int set_identity(cudaStream_t s, int op, void *cell) {
    T v = op == B200ALG_ADD ? Op<T, B200ALG_ADD>::identity() : (op == B200ALG_MAX ? Op<T, B200ALG_MAX>::identity() : Op<T, B200ALG_MIN>::identity());
    set_identity_kernel<T><<<1, 1, 0, s>>>((T *)cell, v);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

// Measurement hook (b200alg_testing_time_sort_mg): events of the calling thread's next sort,
// recorded where one phase ends and the next begins.
constexpr int kSortPhases = 6;
thread_local cudaEvent_t *g_phase_events = nullptr;
static void mark_phase(int boundary, cudaStream_t s) {
    if (g_phase_events) cudaEventRecord(g_phase_events[boundary], s);
}

template <typename K>
static int sort_mg_typed(b200alg_comm *c, cudaStream_t s, const void *keys, const void *values, int64_t n, int key_dtype,
                         int value_bytes, int order, void *out_keys, void *out_values, int64_t out_capacity,
                         int64_t *out_count) {
    const int G = c->ranks;
    const int kb = (int)sizeof(K);
    unsigned char *sc = c->scratch;
    CommState *st = c->state;
    // this rank's mailboxes, filled by everybody (this rank included)
    const long long *all = (const long long *)((const unsigned char *)c->flags + kSampleMailboxAt);
    const long long *matrix = (const long long *)((const unsigned char *)c->flags + kMatrixMailboxAt);
    K *sample_keys = (K *)(sc + c->off_sample_keys);
    long long *sample_index = (long long *)(sc + c->off_sample_index);
    const int64_t total_samples = (int64_t)G * kSamplesPerRank;

    // 1. splitters from (key, position) samples of every shard: every rank stores its samples
    //    into everybody's mailbox; after the barrier they are all there.  (Nobody still reads the
    //    mailboxes of the sort before: a rank gets past that sort's last barrier only when all
    //    ranks have reached it, with their reads behind them in stream order.)
    mark_phase(0, s);
    sample_kernel<K><<<8, 256, 0, s>>>((const K *)keys, n, c->rank, G, c->d_peer_flags);
    B200ALG_LAUNCH_CHECK();
    int rc = rank_barrier(c, s);
    if (rc != B200ALG_OK) return rc;
    collect_samples_kernel<K><<<G, 256, 0, s>>>(all, G, sample_keys, sample_index, &st->sample_count);
    B200ALG_LAUNCH_CHECK();
    // blocks lie in rank order and positions ascend inside a block, so slot order breaks ties the
    // way positions would; the splitters are the pairs of ranks j * count / G, found by counting
    rc = b200alg_select_splitters(s, sample_keys, (const int64_t *)sample_index, total_samples,
                                  (const int64_t *)&st->sample_count, key_dtype, order, G - 1, st->splitter_keys,
                                  (int64_t *)st->splitter_index, sc + c->off_sort_temp, c->sort_temp_bytes);
    if (rc != B200ALG_OK) return rc;

    // 2. bucket sizes of this shard, stored into everybody's matrix
    mark_phase(1, s);
    const long long base = (long long)c->rank << kRankShift;
    rc = b200alg_bucket_count(s, n ? keys : (const void *)sample_keys, n, key_dtype, order, st->splitter_keys, (const int64_t *)st->splitter_index,
                              G - 1, base, (int64_t *)st->bucket_counts, sc + c->off_partition_temp, c->partition_temp_bytes);
    if (rc != B200ALG_OK) return rc;
    publish_counts_kernel<<<1, 32, 0, s>>>(st->bucket_counts, (long long)out_capacity, c->rank, G, c->d_peer_flags);
    B200ALG_LAUNCH_CHECK();

    // 3. the matrix is complete and every rank is done with what the previous sort left in its
    //    receive buffer; each rank works out where its buckets go, then the partition kernel
    //    stores each bucket straight into its owner's buffer
    mark_phase(2, s);
    rc = rank_barrier(c, s);
    if (rc != B200ALG_OK) return rc;
    plan_exchange_kernel<<<1, 32, 0, s>>>(st, matrix, c->d_peer_recv, c->rank, G, (long long)c->capacity, kb, value_bytes,
                                          sc + c->off_sink);
    B200ALG_LAUNCH_CHECK();
    mark_phase(3, s);
    if (n > 0) {
        rc = b200alg_bucket_scatter(s, keys, values, n, key_dtype, value_bytes, order, st->splitter_keys, (const int64_t *)st->splitter_index, G - 1,
                                    base, st->key_ptrs, st->value_ptrs, sc + c->off_partition_temp, c->partition_temp_bytes);
        if (rc != B200ALG_OK) return rc;
    }
    mark_phase(4, s);
    rc = rank_barrier(c, s);  // every rank's stores have landed
    if (rc != B200ALG_OK) return rc;
    mark_phase(5, s);

    // 4. received runs lie in source-rank order; a stable sort straight out of the receive
    //    buffer finishes the job (its length is only known on the device)
    const int64_t bound = c->capacity < out_capacity ? c->capacity : out_capacity;
    if (bound > 0) {
        rc = b200alg_radix_sort_out_of_place(s, c->recv, value_bytes ? c->recv + c->capacity * 8 : nullptr, out_keys, out_values,
                                             bound, (const int64_t *)&st->recv_count, key_dtype, value_bytes, order,
                                             sc + c->off_sort_temp, c->sort_temp_bytes);
        if (rc != B200ALG_OK) return rc;
    }
    B200ALG_CUDA_TRY(cudaMemcpyAsync(out_count, &st->recv_count, 8, cudaMemcpyDeviceToDevice, s));
    mark_phase(6, s);
    return B200ALG_OK;
}

}  // namespace b200alg

using namespace b200alg;

extern "C" int b200alg_comm_unique_id(void *id_bytes) {
    if (!id_bytes) return B200ALG_INVALID_ARGUMENT;
    static_assert(sizeof(ncclUniqueId) <= B200ALG_UNIQUE_ID_BYTES, "unique id size");
    ncclUniqueId id;
    if (ncclGetUniqueId(&id) != ncclSuccess) return B200ALG_NCCL_ERROR;
    memset(id_bytes, 0, B200ALG_UNIQUE_ID_BYTES);
    memcpy(id_bytes, &id, sizeof(id));
    return B200ALG_OK;
}

extern "C" int b200alg_comm_create_rank(const void *id_bytes, int num_ranks, int rank, int64_t sort_capacity, b200alg_comm **out) {
    if (!id_bytes || !out || num_ranks < 1 || num_ranks > kMaxRanks || rank < 0 || rank >= num_ranks) return B200ALG_INVALID_ARGUMENT;
    b200alg_comm *c = new b200alg_comm();
    c->rank = rank;
    c->ranks = num_ranks;
    if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return B200ALG_CUDA_ERROR; }
    ncclUniqueId id;
    memcpy(&id, id_bytes, sizeof(id));
    if (ncclCommInitRank(&c->nccl, num_ranks, id, rank) != ncclSuccess) { delete c; return B200ALG_NCCL_ERROR; }
    const int rc = finish_comm(c, sort_capacity, nullptr);
    if (rc != B200ALG_OK) { b200alg_comm_destroy(c); return rc; }
    *out = c;
    return B200ALG_OK;
}

extern "C" int b200alg_comm_create(int ndev, const int *devs, int64_t sort_capacity, b200alg_comm **out) {
    if (!devs || !out || ndev < 1 || ndev > kMaxRanks) return B200ALG_INVALID_ARGUMENT;
    std::vector<ncclComm_t> comms(ndev);
    if (ncclCommInitAll(comms.data(), ndev, devs) != ncclSuccess) return B200ALG_NCCL_ERROR;
    int before = 0;
    cudaGetDevice(&before);
    for (int i = 0; i < ndev; ++i) {
        out[i] = new b200alg_comm();
        out[i]->rank = i;
        out[i]->ranks = ndev;
        out[i]->device = devs[i];
        out[i]->nccl = comms[i];
    }
    // the handle exchange is a collective that synchronises its stream: one thread per rank
    int rc = B200ALG_OK;
    struct Worker {
        static void *run(void *p) {
            auto *a = (std::pair<b200alg_comm *, int64_t> *)p;
            cudaSetDevice(a->first->device);
            return (void *)(intptr_t)finish_comm(a->first, a->second, nullptr);
        }
    };
    std::vector<pthread_t> threads(ndev);
    std::vector<std::pair<b200alg_comm *, int64_t>> args(ndev);
    for (int i = 0; i < ndev; ++i) {
        args[i] = {out[i], sort_capacity};
        pthread_create(&threads[i], nullptr, Worker::run, &args[i]);
    }
    for (int i = 0; i < ndev; ++i) {
        void *r = nullptr;
        pthread_join(threads[i], &r);
        if ((int)(intptr_t)r != B200ALG_OK) rc = (int)(intptr_t)r;
    }
    cudaSetDevice(before);
    if (rc != B200ALG_OK) {
        for (int i = 0; i < ndev; ++i) { b200alg_comm_destroy(out[i]); out[i] = nullptr; }
    }
    return rc;
}

extern "C" int b200alg_comm_destroy(b200alg_comm *c) {
    if (!c) return B200ALG_OK;
    int before = 0;
    cudaGetDevice(&before);
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < c->ranks; ++r) {
        if (c->opened_recv[r]) cudaIpcCloseMemHandle(c->peer_recv[r]);
        if (c->opened_flags[r]) cudaIpcCloseMemHandle(c->peer_flags[r]);
    }
    if (c->nccl) ncclCommDestroy(c->nccl);
    cudaFree(c->state);
    cudaFree(c->recv);
    cudaFree(c->flags);
    cudaFree(c->scratch);
    cudaFree(c->d_peer_recv);
    cudaFree(c->d_peer_flags);
    cudaSetDevice(before);
    delete c;
    return B200ALG_OK;
}

extern "C" int b200alg_comm_rank(const b200alg_comm *c, int *rank, int *num_ranks) {
    if (!c) return B200ALG_INVALID_ARGUMENT;
    if (rank) *rank = c->rank;
    if (num_ranks) *num_ranks = c->ranks;
    return B200ALG_OK;
}

extern "C" int b200alg_comm_last_nccl_error(const b200alg_comm *c) { return c ? c->last_nccl : 0; }

extern "C" int b200alg_comm_status(b200alg_comm *c, void *stream) {
    if (!c) return B200ALG_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    unsigned int flag = 0;
    B200ALG_CUDA_TRY(cudaMemcpyAsync(&flag, &c->state->hdr.wait_limit_hit, 4, cudaMemcpyDeviceToHost, s));
    B200ALG_CUDA_TRY(cudaStreamSynchronize(s));
    if (flag) {
        B200ALG_CUDA_TRY(cudaMemsetAsync(&c->state->hdr.wait_limit_hit, 0, 4, s));
        return B200ALG_WAIT_LIMIT;
    }
    ncclResult_t async = ncclSuccess;
    if (ncclCommGetAsyncError(c->nccl, &async) != ncclSuccess || async != ncclSuccess) {
        c->last_nccl = (int)async;
        return B200ALG_NCCL_ERROR;
    }
    return B200ALG_OK;
}

extern "C" int b200alg_reduce_mg(b200alg_comm *c, void *stream, const void *in, int64_t stride, int64_t n, int dtype, int op,
                                 void *out) {
    if (!c || !out) return B200ALG_INVALID_ARGUMENT;
    ncclDataType_t t;
    if (!nccl_type(dtype, &t)) return B200ALG_UNSUPPORTED;
    if (op < B200ALG_ADD || op > B200ALG_MIN) return B200ALG_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (n > 0) {
        rc = b200alg_reduce(s, in, stride, n, dtype, op, out);
    } else {  // an empty shard contributes the identity
        switch (dtype) {
        case B200ALG_I32: rc = set_identity<int32_t>(s, op, out); break;
        case B200ALG_U32: rc = set_identity<uint32_t>(s, op, out); break;
        case B200ALG_I64: rc = set_identity<int64_t>(s, op, out); break;
        case B200ALG_U64: rc = set_identity<uint64_t>(s, op, out); break;
        case B200ALG_F32: rc = set_identity<float>(s, op, out); break;
        default: rc = set_identity<double>(s, op, out); break;
        }
    }
    if (rc != B200ALG_OK) return rc;
    B200ALG_NCCL_TRY(c, ncclAllReduce(out, out, 1, t, nccl_op(op), c->nccl, s));
    return B200ALG_OK;
}

extern "C" int b200alg_histogram_mg(b200alg_comm *c, void *stream, const void *in, int64_t stride, int64_t n, int in_dtype,
                                    int locator, double lo, double hi, void *bins, int64_t num_bins, int bin_dtype,
                                    void *overflow) {
    if (!c || !bins || num_bins < 1) return B200ALG_INVALID_ARGUMENT;
    ncclDataType_t t;
    if (!nccl_type(bin_dtype, &t)) return B200ALG_UNSUPPORTED;
    const int bb = dtype_bytes(bin_dtype);
    if (num_bins * bb > (1 << 20)) return B200ALG_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    void *local = c->scratch + c->off_bins;
    B200ALG_CUDA_TRY(cudaMemsetAsync(local, 0, (size_t)(num_bins * bb), s));
    if (n > 0) {
        const int rc = b200alg_histogram(s, in, stride, n, in_dtype, locator, lo, hi, local, num_bins, bin_dtype, nullptr);
        if (rc != B200ALG_OK) return rc;
    }
    B200ALG_NCCL_TRY(c, ncclAllReduce(local, local, (size_t)num_bins, t, ncclSum, c->nccl, s));
    const int blocks = (int)((num_bins + 255) / 256 > 64 ? 64 : (num_bins + 255) / 256);
    add_bins_kernel<<<blocks, 256, 0, s>>>(bins, local, num_bins, bin_dtype, (int *)overflow);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

extern "C" int b200alg_scan_mg(b200alg_comm *c, void *stream, const void *in, void *out, int64_t n, int dtype, int op,
                               int inclusive, void *temp, int64_t temp_bytes) {
    if (!c) return B200ALG_INVALID_ARGUMENT;
    ncclDataType_t t;
    if (!nccl_type(dtype, &t)) return B200ALG_UNSUPPORTED;
    if (op < B200ALG_ADD || op > B200ALG_MIN) return B200ALG_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    CommState *st = c->state;
    void *total = &st->scalar[0], *carry = &st->scalar[2];
    // total of this shard (identity when it is empty), everybody's totals, fold of the lower ranks'
    int rc;
    if (n > 0) {
        rc = b200alg_reduce(s, in, 1, n, dtype, op, total);
    } else {
        switch (dtype) {
        case B200ALG_I32: rc = set_identity<int32_t>(s, op, total); break;
        case B200ALG_U32: rc = set_identity<uint32_t>(s, op, total); break;
        case B200ALG_I64: rc = set_identity<int64_t>(s, op, total); break;
        case B200ALG_U64: rc = set_identity<uint64_t>(s, op, total); break;
        case B200ALG_F32: rc = set_identity<float>(s, op, total); break;
        default: rc = set_identity<double>(s, op, total); break;
        }
    }
    if (rc != B200ALG_OK) return rc;
    B200ALG_NCCL_TRY(c, ncclAllGather(total, st->gathered, 1, t, c->nccl, s));
    switch (dtype) {
    case B200ALG_I32: rc = fold_lower<int32_t>(s, op, st->gathered, c->rank, carry); break;
    case B200ALG_U32: rc = fold_lower<uint32_t>(s, op, st->gathered, c->rank, carry); break;
    case B200ALG_I64: rc = fold_lower<int64_t>(s, op, st->gathered, c->rank, carry); break;
    case B200ALG_U64: rc = fold_lower<uint64_t>(s, op, st->gathered, c->rank, carry); break;
    case B200ALG_F32: rc = fold_lower<float>(s, op, st->gathered, c->rank, carry); break;
    default: rc = fold_lower<double>(s, op, st->gathered, c->rank, carry); break;
    }
    if (rc != B200ALG_OK) return rc;
    if (n == 0) return B200ALG_OK;
    return b200alg_scan_carry(s, in, 1, out, 1, n, dtype, op, inclusive, carry, temp, temp_bytes);
}

extern "C" int b200alg_sort_mg(b200alg_comm *c, void *stream, const void *keys, const void *values, int64_t n, int key_dtype,
                               int value_bytes, int order, void *out_keys, void *out_values, int64_t out_capacity,
                               int64_t *out_count) {
    if (!c || !out_keys || !out_count || n < 0 || out_capacity < 0) return B200ALG_INVALID_ARGUMENT;
    if ((n > 0 && !keys) || (value_bytes && n > 0 && !values) || (value_bytes && !out_values)) return B200ALG_INVALID_ARGUMENT;
    if (value_bytes != 0 && value_bytes != 4 && value_bytes != 8) return B200ALG_UNSUPPORTED;
    if (c->capacity <= 0) return B200ALG_TEMP_TOO_SMALL;   // created without a sort capacity
    if (n > c->capacity) return B200ALG_TEMP_TOO_SMALL;
    if ((uintptr_t)out_count % 8) return B200ALG_MISALIGNED;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype_bytes(key_dtype)) {
    case 1: return sort_mg_typed<uint8_t>(c, s, keys, values, n, key_dtype, value_bytes, order, out_keys, out_values, out_capacity, out_count);
    case 2: return sort_mg_typed<uint16_t>(c, s, keys, values, n, key_dtype, value_bytes, order, out_keys, out_values, out_capacity, out_count);
    case 4: return sort_mg_typed<uint32_t>(c, s, keys, values, n, key_dtype, value_bytes, order, out_keys, out_values, out_capacity, out_count);
    case 8: return sort_mg_typed<uint64_t>(c, s, keys, values, n, key_dtype, value_bytes, order, out_keys, out_values, out_capacity, out_count);
    }
    return B200ALG_UNSUPPORTED;
}

extern "C" int b200alg_testing_time_sort_mg(b200alg_comm *c, void *stream, const void *keys, const void *values, int64_t n,
                                            int key_dtype, int value_bytes, int order, void *out_keys, void *out_values,
                                            int64_t out_capacity, int64_t *out_count, float *phase_ms) {
    if (!phase_ms) return B200ALG_INVALID_ARGUMENT;
    cudaEvent_t ev[kSortPhases + 1];
    for (int i = 0; i <= kSortPhases; ++i) B200ALG_CUDA_TRY(cudaEventCreate(&ev[i]));
    g_phase_events = ev;
    const int rc = b200alg_sort_mg(c, stream, keys, values, n, key_dtype, value_bytes, order, out_keys, out_values,
                                   out_capacity, out_count);
    g_phase_events = nullptr;
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (rc == B200ALG_OK && e == cudaSuccess) {
        for (int i = 0; i < kSortPhases; ++i)
            if (cudaEventElapsedTime(&phase_ms[i], ev[i], ev[i + 1]) != cudaSuccess) phase_ms[i] = -1.f;
    }
    for (int i = 0; i <= kSortPhases; ++i) cudaEventDestroy(ev[i]);
    if (rc != B200ALG_OK) return rc;
    return e == cudaSuccess ? B200ALG_OK : B200ALG_CUDA_ERROR;
}
