// Histogram: per-block privatised bins in shared memory, replicated per lane so that the
// shared-memory atomics of a warp fall into distinct banks, flushed with one global atomic
// per non-empty bin.
// Replaces HistogramWorkKernel (HistogramExtensions.cs:237-277), which issues one global
// atomic per element, and the overflow reporting of HistogramKernel (:176-198) with
// HistogramIncrement* (HistogramOperations.tt:30-41).
#include "common.cuh"

namespace b200alg {

constexpr int kHistThreads = 512;
constexpr int kHistWarps = kHistThreads / 32;
constexpr int64_t kHistSmemBytes = 48 * 1024;  // static limit, no opt-in needed

struct LocParams {
    double lo_d, scale_d, bins_d;  // bins_* = num_bins as a floating-point value
    float lo_f, scale_f, bins_f;
    long long num_bins;
    int last;  // num_bins - 1
};

// ---- bin locators ---------------------------------------------------------------------
// run() returns the bin as an int (the bin count is below 2^31); kInRange = the result needs
// no bounds check.
template <typename T, int LOCATOR> struct Locate;

template <> struct Locate<float, B200ALG_LOCATOR_EQUAL_WIDTH_CLAMP> {
    static constexpr bool kInRange = true;
    static __device__ __forceinline__ int run(float x, const LocParams &p) {
        // floor, then clamp == clamp, then truncate; fmaxf(NaN, 0) = 0 sends NaN to bin 0
        const float t = fminf(fmaxf((x - p.lo_f) * p.scale_f, 0.0f), p.bins_f);
        return min(__float2int_rz(t), p.last);
    }
};
template <typename T> struct Locate<T, B200ALG_LOCATOR_EQUAL_WIDTH_CLAMP> {
    static constexpr bool kInRange = true;
    static __device__ __forceinline__ int run(T x, const LocParams &p) {
        const double t = fmin(fmax(((double)x - p.lo_d) * p.scale_d, 0.0), p.bins_d);
        return min(__double2int_rz(t), p.last);
    }
};
template <> struct Locate<int32_t, B200ALG_LOCATOR_MODULO> {
    static constexpr bool kInRange = true;
    static __device__ __forceinline__ int run(int32_t x, const LocParams &p) {
        const int r = x % (int)p.num_bins;
        return r < 0 ? -r : r;
    }
};
template <> struct Locate<int64_t, B200ALG_LOCATOR_MODULO> {
    static constexpr bool kInRange = true;
    static __device__ __forceinline__ int run(int64_t x, const LocParams &p) {
        const long long r = (long long)x % p.num_bins;
        return (int)(r < 0 ? -r : r);
    }
};
template <> struct Locate<uint32_t, B200ALG_LOCATOR_MODULO> {
    static constexpr bool kInRange = true;
    static __device__ __forceinline__ int run(uint32_t x, const LocParams &p) { return (int)(x % (unsigned int)p.num_bins); }
};
template <> struct Locate<uint64_t, B200ALG_LOCATOR_MODULO> {
    static constexpr bool kInRange = true;
    static __device__ __forceinline__ int run(uint64_t x, const LocParams &p) {
        return (int)(x % (unsigned long long)p.num_bins);
    }
};
template <> struct Locate<float, B200ALG_LOCATOR_MODULO> {
    static constexpr bool kInRange = false;
    static __device__ __forceinline__ int run(float x, const LocParams &p) {
        return (int)fabsf(fmodf(x, (float)p.num_bins));
    }
};
template <> struct Locate<double, B200ALG_LOCATOR_MODULO> {
    static constexpr bool kInRange = false;
    static __device__ __forceinline__ int run(double x, const LocParams &p) {
        return (int)fabs(fmod(x, (double)p.num_bins));
    }
};

// ---- adding a block's count to a global bin --------------------------------------------
// The reference raises the overflow flag when some single increment starts from
// MaxValue.  Adding c at once starts from old, old+1, ..., old+c-1 (wrapping), so the flag
// is raised iff the distance from old up to MaxValue is below c.
__device__ __forceinline__ bool add_to_bin(void *bins, long long b, unsigned long long c, int bin_dtype) {
    switch (bin_dtype) {
    case B200ALG_I32: {
        unsigned int old = atomicAdd((unsigned int *)bins + b, (unsigned int)c);
        return (unsigned long long)(unsigned int)(0x7FFFFFFFu - old) < c;
    }
    case B200ALG_U32: {
        unsigned int old = atomicAdd((unsigned int *)bins + b, (unsigned int)c);
        return (unsigned long long)(unsigned int)(0xFFFFFFFFu - old) < c;
    }
    case B200ALG_I64: {
        unsigned long long old = atomicAdd((unsigned long long *)bins + b, c);
        return (0x7FFFFFFFFFFFFFFFull - old) < c;
    }
    case B200ALG_U64: {
        unsigned long long old = atomicAdd((unsigned long long *)bins + b, c);
        return (0xFFFFFFFFFFFFFFFFull - old) < c;
    }
    case B200ALG_F32: {
        float old = atomicAdd((float *)bins + b, (float)c);
        return old == FLT_MAX;
    }
    default: {
        double old = atomicAdd((double *)bins + b, (double)c);
        return old == DBL_MAX;
    }
    }
}

// ---- shared-memory privatised kernel ---------------------------------------------------
template <typename T, int LOCATOR, bool VECTOR>
__global__ void __launch_bounds__(kHistThreads)
histogram_smem_kernel(const T *__restrict__ in, int64_t stride, int64_t n, LocParams p, void *bins, int bin_dtype,
                      int *overflow, int replicas) {
    // Bin b has `replicas` (a power of two, up to 32) counters at sh[b * replicas + r]; lane l
    // uses r = l % replicas.  With 32 replicas every lane of a warp has a bank of its own, so
    // an atomic instruction is one wavefront whatever the distribution of the data.
    extern __shared__ unsigned int sh[];
    const int nb = (int)p.num_bins;
    for (int i = threadIdx.x; i < nb * replicas; i += kHistThreads) sh[i] = 0u;
    __syncthreads();

    unsigned int *mine = sh + (threadIdx.x & (replicas - 1));
    const int rshift = 31 - __clz(replicas);
    const int64_t step = (int64_t)gridDim.x * kHistThreads;
    const int64_t gtid = (int64_t)blockIdx.x * kHistThreads + threadIdx.x;

    if (VECTOR) {
        constexpr int VEC = 16 / sizeof(T);
        union V { uint4 u; T t[VEC]; };
        int64_t head = (int64_t)(((16u - (unsigned)((uintptr_t)in & 15u)) & 15u) / sizeof(T));
        if (head > n) head = n;
        const uint4 *vin = reinterpret_cast<const uint4 *>(in + head);
        const int64_t nvec = (n - head) / VEC;
        const int64_t tail = head + nvec * VEC;
        int64_t i = gtid;
        for (; i + step < nvec; i += 2 * step) {
            V a, b;
            a.u = __ldcs(vin + i);
            b.u = __ldcs(vin + i + step);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                const int ba = Locate<T, LOCATOR>::run(a.t[k], p);
                if (Locate<T, LOCATOR>::kInRange || (unsigned int)ba < (unsigned int)nb) atomicAdd(mine + (ba << rshift), 1u);
            }
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                const int bb = Locate<T, LOCATOR>::run(b.t[k], p);
                if (Locate<T, LOCATOR>::kInRange || (unsigned int)bb < (unsigned int)nb) atomicAdd(mine + (bb << rshift), 1u);
            }
        }
        for (; i < nvec; i += step) {
            V a;
            a.u = __ldcs(vin + i);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                const int ba = Locate<T, LOCATOR>::run(a.t[k], p);
                if (Locate<T, LOCATOR>::kInRange || (unsigned int)ba < (unsigned int)nb) atomicAdd(mine + (ba << rshift), 1u);
            }
        }
        if (blockIdx.x == 0) {
            for (int64_t j = threadIdx.x; j < head; j += kHistThreads) {
                const int b = Locate<T, LOCATOR>::run(in[j], p);
                if (Locate<T, LOCATOR>::kInRange || (unsigned int)b < (unsigned int)nb) atomicAdd(mine + (b << rshift), 1u);
            }
            for (int64_t j = tail + threadIdx.x; j < n; j += kHistThreads) {
                const int b = Locate<T, LOCATOR>::run(in[j], p);
                if (Locate<T, LOCATOR>::kInRange || (unsigned int)b < (unsigned int)nb) atomicAdd(mine + (b << rshift), 1u);
            }
        }
    } else {
        for (int64_t i = gtid; i < n; i += step) {
            const int b = Locate<T, LOCATOR>::run(in[i * stride], p);
            if (Locate<T, LOCATOR>::kInRange || (unsigned int)b < (unsigned int)nb) atomicAdd(mine + (b << rshift), 1u);
        }
    }
    __syncthreads();

    bool of = false;
    for (int b = threadIdx.x; b < nb; b += kHistThreads) {
        unsigned long long c = 0;
        for (int r = 0; r < replicas; ++r) c += sh[b * replicas + ((r + threadIdx.x) & (replicas - 1))];
        if (c) of |= add_to_bin(bins, b, c, bin_dtype);
    }
    if (overflow && __syncthreads_or(of) && threadIdx.x == 0) atomicOr(overflow, 1);
}

// ---- fallback for bin counts that do not fit in shared memory ---------------------------
template <typename T, int LOCATOR>
__global__ void __launch_bounds__(256)
histogram_global_kernel(const T *__restrict__ in, int64_t stride, int64_t n, LocParams p, void *bins, int bin_dtype,
                        int *overflow) {
    bool of = false;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        const int b = Locate<T, LOCATOR>::run(in[i * stride], p);
        if (Locate<T, LOCATOR>::kInRange || (unsigned int)b < (unsigned int)p.num_bins) of |= add_to_bin(bins, b, 1ull, bin_dtype);
    }
    if (overflow && __syncthreads_or(of) && threadIdx.x == 0) atomicOr(overflow, 1);
}

template <typename T, int LOCATOR>
static int launch_histogram(cudaStream_t s, const void *in, int64_t stride, int64_t n, const LocParams &p, void *bins,
                            int bin_dtype, void *overflow) {
    const int64_t nb = p.num_bins;
    if (nb * 4 <= kHistSmemBytes) {
        int replicas = 1;
        while (replicas < 32 && (int64_t)replicas * 2 * nb * 4 <= kHistSmemBytes) replicas *= 2;
        const size_t smem = (size_t)replicas * nb * 4;
        constexpr int VEC = 16 / sizeof(T);
        const int64_t per_block = (int64_t)kHistThreads * (stride == 1 ? VEC * 2 : 2);
        int64_t want = ceil_div(n, per_block);
        const int64_t cap = (int64_t)sm_count() * (2048 / kHistThreads);
        const int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
        if (stride == 1)
            histogram_smem_kernel<T, LOCATOR, true><<<blocks, kHistThreads, smem, s>>>((const T *)in, 1, n, p, bins, bin_dtype, (int *)overflow, replicas);
        else
            histogram_smem_kernel<T, LOCATOR, false><<<blocks, kHistThreads, smem, s>>>((const T *)in, stride, n, p, bins, bin_dtype, (int *)overflow, replicas);
    } else {
        int64_t want = ceil_div(n, 256 * 4);
        const int64_t cap = (int64_t)sm_count() * 8;
        const int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
        histogram_global_kernel<T, LOCATOR><<<blocks, 256, 0, s>>>((const T *)in, stride, n, p, bins, bin_dtype, (int *)overflow);
    }
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

template <typename T>
static int dispatch_locator(cudaStream_t s, const void *in, int64_t stride, int64_t n, int locator, const LocParams &p,
                            void *bins, int bin_dtype, void *overflow) {
    switch (locator) {
    case B200ALG_LOCATOR_EQUAL_WIDTH_CLAMP:
        return launch_histogram<T, B200ALG_LOCATOR_EQUAL_WIDTH_CLAMP>(s, in, stride, n, p, bins, bin_dtype, overflow);
    case B200ALG_LOCATOR_MODULO:
        return launch_histogram<T, B200ALG_LOCATOR_MODULO>(s, in, stride, n, p, bins, bin_dtype, overflow);
    }
    return B200ALG_UNSUPPORTED;
}

}  // namespace b200alg

using namespace b200alg;

extern "C" int b200alg_histogram(void *stream, const void *in, int64_t stride, int64_t n, int in_dtype, int locator,
                                 double lo, double hi, void *bins, int64_t num_bins, int bin_dtype, void *overflow) {
    // Argument checks mirror CreateHistogram's (HistogramExtensions.cs:322-338).
    if (!in || !bins) return B200ALG_INVALID_ARGUMENT;
    if (n < 0 || stride < 1 || num_bins < 1) return B200ALG_INVALID_ARGUMENT;
    if (!is_atomic_numeric(in_dtype) || !is_atomic_numeric(bin_dtype)) return B200ALG_UNSUPPORTED;
    if (n > kMaxElements || num_bins > INT32_MAX) return B200ALG_TOO_LARGE;
    if (locator == B200ALG_LOCATOR_EQUAL_WIDTH_CLAMP && !(hi > lo)) return B200ALG_INVALID_ARGUMENT;
    if (((uintptr_t)in % dtype_bytes(in_dtype)) || ((uintptr_t)bins % dtype_bytes(bin_dtype)) ||
        (overflow && ((uintptr_t)overflow % 4)))
        return B200ALG_MISALIGNED;
    if (n == 0) return B200ALG_OK;
    LocParams p;
    p.num_bins = num_bins;
    p.lo_d = lo;
    p.scale_d = (double)num_bins / (hi - lo);
    p.lo_f = (float)lo;
    p.scale_f = (float)num_bins / ((float)hi - (float)lo);
    p.bins_d = (double)num_bins;
    p.bins_f = (float)num_bins;
    p.last = (int)(num_bins - 1);
    // float input computes in float: a range that collapses or overflows there would put every
    // element into an edge bin without a word
    if (locator == B200ALG_LOCATOR_EQUAL_WIDTH_CLAMP && in_dtype == B200ALG_F32 &&
        (!isfinite((float)lo) || !isfinite((float)hi) || !((float)hi > (float)lo) || !isfinite(p.scale_f) || !(p.scale_f > 0.0f)))
        return B200ALG_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    switch (in_dtype) {
    case B200ALG_I32: return dispatch_locator<int32_t>(s, in, stride, n, locator, p, bins, bin_dtype, overflow);
    case B200ALG_U32: return dispatch_locator<uint32_t>(s, in, stride, n, locator, p, bins, bin_dtype, overflow);
    case B200ALG_I64: return dispatch_locator<int64_t>(s, in, stride, n, locator, p, bins, bin_dtype, overflow);
    case B200ALG_U64: return dispatch_locator<uint64_t>(s, in, stride, n, locator, p, bins, bin_dtype, overflow);
    case B200ALG_F32: return dispatch_locator<float>(s, in, stride, n, locator, p, bins, bin_dtype, overflow);
    case B200ALG_F64: return dispatch_locator<double>(s, in, stride, n, locator, p, bins, bin_dtype, overflow);
    }
    return B200ALG_UNSUPPORTED;
}
