// Unique: removes consecutive duplicates in place and reports how many elements are left.
// Replaces UniqueKernel / CreateUnique (UniqueExtensions.cs:59-195), whose groups run one after
// the other (SequentialGroupExecutor) and whose first thread compacts a whole tile alone.
// Here every tile flags the elements that differ from their left neighbour, chains its count
// to the previous tiles with decoupled look-back, and writes its survivors to scratch; a second
// kernel copies the survivors back.  Equality follows Comparison{T} = first.CompareTo(second)
// (ComparisonOperations.tt): integers compare by value; floating-point values compare equal when
// they are numerically equal or both NaN.
#include "common.cuh"
#include "lookback.cuh"

namespace b200alg {

constexpr int kUniqueThreads = 256;
constexpr int kUniqueItems = 16;
constexpr int kUniqueTile = kUniqueThreads * kUniqueItems;

template <typename T> struct SameValue {
    static __device__ __forceinline__ bool eq(T a, T b) { return a == b; }
};
template <> struct SameValue<float> {
    static __device__ __forceinline__ bool eq(float a, float b) { return a == b || (a != a && b != b); }
};
template <> struct SameValue<double> {
    static __device__ __forceinline__ bool eq(double a, double b) { return a == b || (a != a && b != b); }
};
template <> struct SameValue<__half> {
    static __device__ __forceinline__ bool eq(__half a, __half b) {
        const float x = __half2float(a), y = __half2float(b);
        return x == y || (x != x && y != y);
    }
};

template <typename T>
__global__ void __launch_bounds__(kUniqueThreads)
unique_select_kernel(const T *__restrict__ in, int64_t n, T *__restrict__ kept, long long *__restrict__ starts,
                     long long *out_count, TempHeader *hdr, void *state_base, int num_tiles) {
    __shared__ unsigned int warp_total[kUniqueThreads / 32];
    __shared__ unsigned int warp_excl[kUniqueThreads / 32];
    __shared__ unsigned int s_prefix;
    __shared__ int s_tile;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_tile = (int)atomicAdd(&hdr->reserved[0], 1u);  // tiles are handed out in order
    __syncthreads();
    const int tile = s_tile;
    const int64_t first = (int64_t)tile * kUniqueTile + (int64_t)tid * kUniqueItems;

    // thread t owns kUniqueItems consecutive elements; keep[k] = element k starts a new run
    T item[kUniqueItems];
    T left = T();
    const bool has_left = first > 0 && first < n;
    if (has_left) left = in[first - 1];
    unsigned int keep_mask = 0u, count = 0u;
#pragma unroll
    for (int k = 0; k < kUniqueItems; ++k) {
        const int64_t idx = first + k;
        if (idx < n) {
            item[k] = in[idx];
            const bool keep = (idx == 0) || !SameValue<T>::eq(item[k], k == 0 ? left : item[k - 1]);
            keep_mask |= (unsigned int)keep << k;
            count += keep;
        }
    }

    // block scan of the per-thread counts
    unsigned int incl = count;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) warp_total[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        unsigned int wt = lane < kUniqueThreads / 32 ? warp_total[lane] : 0u;
        unsigned int wi = wt;
#pragma unroll
        for (int d = 1; d < kUniqueThreads / 32; d <<= 1) {
            const unsigned int up = __shfl_up_sync(0xffffffffu, wi, d);
            if (lane >= d) wi += up;
        }
        if (lane < kUniqueThreads / 32) warp_excl[lane] = wi - wt;
        const unsigned int aggregate = __shfl_sync(0xffffffffu, wi, kUniqueThreads / 32 - 1);

        TileState<unsigned int> state(state_base, num_tiles);
        unsigned int prefix = 0u;
        if (tile == 0) {
            if (lane == 0) state.publish(0, kInclusive, aggregate);
        } else {
            if (lane == 0) state.publish(tile, kAggregate, aggregate);
            int look = tile - 1 - lane;  // 32 predecessors per round, nearest first
            bool gave_up = false;
            while (true) {
                unsigned int v = 0u;
                unsigned int flag = kInclusive;
                if (look >= 0) {
                    unsigned int spins = 0;
                    flag = state.poll(look, v);
                    while (flag == kInvalid) {
                        if (++spins > kMaxSpin) { gave_up = true; flag = kInclusive; v = 0u; break; }
                        __nanosleep(20);
                        flag = state.poll(look, v);
                    }
                }
                const unsigned int incl_mask = __ballot_sync(0xffffffffu, flag == kInclusive);
                const int nearest = incl_mask ? (__ffs(incl_mask) - 1) : 31;
                unsigned int contrib = lane <= nearest ? v : 0u;
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) contrib += __shfl_down_sync(0xffffffffu, contrib, d);
                prefix += __shfl_sync(0xffffffffu, contrib, 0);
                if (incl_mask) break;
                look -= 32;
            }
            if (__any_sync(0xffffffffu, gave_up) && lane == 0) atomicExch(&hdr->wait_limit_hit, 1u);
            if (lane == 0) state.publish(tile, kInclusive, prefix + aggregate);
        }
        if (lane == 0) {
            s_prefix = prefix;
            if (tile == num_tiles - 1) *out_count = (long long)prefix + aggregate;
        }
    }
    __syncthreads();

    unsigned int pos = s_prefix + warp_excl[warp] + (incl - count);
#pragma unroll
    for (int k = 0; k < kUniqueItems; ++k) {
        if ((keep_mask >> k) & 1u) {
            kept[pos] = item[k];
            if (starts) starts[pos] = first + k;  // where the run begins (run-length encoding)
            ++pos;
        }
    }
}

// lengths[r] = distance from the start of run r to the start of the next run (or to n).
__global__ void __launch_bounds__(256)
run_lengths_kernel(const long long *starts, const long long *count, long long n, long long *lengths) {
    const long long m = *count;
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < m; r += step)
        lengths[r] = (r + 1 < m ? starts[r + 1] : n) - starts[r];
}

template <typename T>
__global__ void __launch_bounds__(256)
unique_copy_back_kernel(T *data, const T *kept, const long long *count) {
    const long long m = *count;
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += step) data[i] = kept[i];
}

struct UniqueLayout {
    int64_t tiles, off_state, off_kept, total;
};

static UniqueLayout unique_layout(int elem_bytes, int64_t n) {
    UniqueLayout L;
    L.tiles = ceil_div(n < 1 ? 1 : n, kUniqueTile);
    L.off_state = sizeof(TempHeader);
    L.off_kept = L.off_state + round_up(L.tiles * kDescStride, 256);
    L.total = L.off_kept + round_up((n < 1 ? 1 : n) * elem_bytes, 256);
    return L;
}

template <typename T>
static int run_unique(cudaStream_t s, void *data, int64_t n, void *out_count, void *temp, const UniqueLayout &L) {
    char *t = (char *)temp;
    B200ALG_CUDA_TRY(cudaMemsetAsync(temp, 0, (size_t)L.off_kept, s));
    unique_select_kernel<T><<<(int)L.tiles, kUniqueThreads, 0, s>>>((const T *)data, n, (T *)(t + L.off_kept), nullptr,
                                                                  (long long *)out_count, (TempHeader *)temp, t + L.off_state,
                                                                  (int)L.tiles);
    B200ALG_LAUNCH_CHECK();
    int64_t want = ceil_div(n, 256 * 8);
    const int64_t cap = (int64_t)sm_count() * 8;
    const int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    unique_copy_back_kernel<T><<<blocks, 256, 0, s>>>((T *)data, (const T *)(t + L.off_kept), (const long long *)out_count);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

// Run-length encoding: the same selection, with the survivors written to the caller's array
// and the run starts to scratch, from which the lengths follow.
struct RunLengthLayout {
    int64_t tiles, off_state, off_starts, total;
};
static RunLengthLayout run_length_layout(int64_t n) {
    RunLengthLayout L;
    L.tiles = ceil_div(n < 1 ? 1 : n, kUniqueTile);
    L.off_state = sizeof(TempHeader);
    L.off_starts = L.off_state + round_up(L.tiles * kDescStride, 256);
    L.total = L.off_starts + round_up((n < 1 ? 1 : n) * 8, 256);
    return L;
}

template <typename T>
static int run_rle(cudaStream_t s, const void *data, int64_t n, void *values, void *lengths, void *num_runs, void *temp,
                   const RunLengthLayout &L) {
    char *t = (char *)temp;
    B200ALG_CUDA_TRY(cudaMemsetAsync(temp, 0, (size_t)L.off_starts, s));
    unique_select_kernel<T><<<(int)L.tiles, kUniqueThreads, 0, s>>>((const T *)data, n, (T *)values, (long long *)(t + L.off_starts),
                                                                  (long long *)num_runs, (TempHeader *)temp, t + L.off_state,
                                                                  (int)L.tiles);
    B200ALG_LAUNCH_CHECK();
    int64_t want = ceil_div(n, 256 * 8);
    const int64_t cap = (int64_t)sm_count() * 8;
    const int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    run_lengths_kernel<<<blocks, 256, 0, s>>>((const long long *)(t + L.off_starts), (const long long *)num_runs, (long long)n,
                                              (long long *)lengths);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

}  // namespace b200alg

using namespace b200alg;

extern "C" int b200alg_run_length_encode_temp_bytes(int dtype, int64_t n, int64_t *out_bytes) {
    if (!out_bytes || n < 0) return B200ALG_INVALID_ARGUMENT;
    if (dtype_bytes(dtype) == 0) return B200ALG_UNSUPPORTED;
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
    *out_bytes = run_length_layout(n).total;
    return B200ALG_OK;
}

extern "C" int b200alg_run_length_encode(void *stream, const void *data, int64_t n, int dtype, void *values, int64_t *lengths,
                                         int64_t *num_runs, void *temp, int64_t temp_bytes) {
    if (!num_runs || n < 0) return B200ALG_INVALID_ARGUMENT;
    if ((uintptr_t)num_runs % 8) return B200ALG_MISALIGNED;
    if (n == 0) {
        B200ALG_CUDA_TRY(cudaMemsetAsync(num_runs, 0, 8, (cudaStream_t)stream));
        return B200ALG_OK;
    }
    if (!data || !values || !lengths || !temp) return B200ALG_INVALID_ARGUMENT;
    const int es = dtype_bytes(dtype);
    if (es == 0) return B200ALG_UNSUPPORTED;
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
    if (((uintptr_t)data % es) || ((uintptr_t)values % es) || ((uintptr_t)lengths % 8) || ((uintptr_t)temp % 256)) return B200ALG_MISALIGNED;
    const RunLengthLayout L = run_length_layout(n);
    if (temp_bytes < L.total) return B200ALG_TEMP_TOO_SMALL;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case B200ALG_I8: case B200ALG_U8: return run_rle<uint8_t>(s, data, n, values, lengths, num_runs, temp, L);
    case B200ALG_I16: case B200ALG_U16: return run_rle<uint16_t>(s, data, n, values, lengths, num_runs, temp, L);
    case B200ALG_I32: case B200ALG_U32: return run_rle<uint32_t>(s, data, n, values, lengths, num_runs, temp, L);
    case B200ALG_I64: case B200ALG_U64: return run_rle<uint64_t>(s, data, n, values, lengths, num_runs, temp, L);
    case B200ALG_F16: return run_rle<__half>(s, data, n, values, lengths, num_runs, temp, L);
    case B200ALG_F32: return run_rle<float>(s, data, n, values, lengths, num_runs, temp, L);
    case B200ALG_F64: return run_rle<double>(s, data, n, values, lengths, num_runs, temp, L);
    }
    return B200ALG_UNSUPPORTED;
}

extern "C" int b200alg_unique_temp_bytes(int dtype, int64_t n, int64_t *out_bytes) {
    if (!out_bytes || n < 0) return B200ALG_INVALID_ARGUMENT;
    const int es = dtype_bytes(dtype);
    if (es == 0) return B200ALG_UNSUPPORTED;
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
    *out_bytes = unique_layout(es, n).total;
    return B200ALG_OK;
}

extern "C" int b200alg_unique(void *stream, void *data, int64_t n, int dtype, void *out_count, void *temp, int64_t temp_bytes) {
    // Argument checks mirror CreateUnique's (UniqueExtensions.cs:150-172).
    if (!out_count || n < 0) return B200ALG_INVALID_ARGUMENT;
    if ((uintptr_t)out_count % 8) return B200ALG_MISALIGNED;
    if (n == 0) {  // an empty view has no address
        B200ALG_CUDA_TRY(cudaMemsetAsync(out_count, 0, 8, (cudaStream_t)stream));
        return B200ALG_OK;
    }
    if (!data || !temp) return B200ALG_INVALID_ARGUMENT;
    const int es = dtype_bytes(dtype);
    if (es == 0) return B200ALG_UNSUPPORTED;
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
    if (((uintptr_t)data % es) || ((uintptr_t)out_count % 8) || ((uintptr_t)temp % 256)) return B200ALG_MISALIGNED;
    const UniqueLayout L = unique_layout(es, n);
    if (temp_bytes < L.total) return B200ALG_TEMP_TOO_SMALL;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case B200ALG_I8: case B200ALG_U8: return run_unique<uint8_t>(s, data, n, out_count, temp, L);
    case B200ALG_I16: case B200ALG_U16: return run_unique<uint16_t>(s, data, n, out_count, temp, L);
    case B200ALG_I32: case B200ALG_U32: return run_unique<uint32_t>(s, data, n, out_count, temp, L);
    case B200ALG_I64: case B200ALG_U64: return run_unique<uint64_t>(s, data, n, out_count, temp, L);
    case B200ALG_F16: return run_unique<__half>(s, data, n, out_count, temp, L);
    case B200ALG_F32: return run_unique<float>(s, data, n, out_count, temp, L);
    case B200ALG_F64: return run_unique<double>(s, data, n, out_count, temp, L);
    }
    return B200ALG_UNSUPPORTED;
}
