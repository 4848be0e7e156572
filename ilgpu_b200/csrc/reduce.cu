// Reduce: grid-stride fold with 128-bit loads, warp-shuffle tree, one atomic per block.
// Replaces ReductionImplementation + CreateReduction (ReductionExtensions.cs:52-167).
#include "common.cuh"

namespace b200alg {

// AtomicApply of IScanReduceOperation<T> (ScanReduceOperations.tt:66-70).
template <typename T, int OP> struct AtomicApply;

template <> struct AtomicApply<int32_t, B200ALG_ADD> { static __device__ void run(int32_t *p, int32_t v) { atomicAdd((unsigned int *)p, (unsigned int)v); } };
template <> struct AtomicApply<uint32_t, B200ALG_ADD> { static __device__ void run(uint32_t *p, uint32_t v) { atomicAdd(p, v); } };
template <> struct AtomicApply<int64_t, B200ALG_ADD> { static __device__ void run(int64_t *p, int64_t v) { atomicAdd((unsigned long long *)p, (unsigned long long)v); } };
template <> struct AtomicApply<uint64_t, B200ALG_ADD> { static __device__ void run(uint64_t *p, uint64_t v) { atomicAdd((unsigned long long *)p, (unsigned long long)v); } };
template <> struct AtomicApply<float, B200ALG_ADD> { static __device__ void run(float *p, float v) { atomicAdd(p, v); } };
template <> struct AtomicApply<double, B200ALG_ADD> { static __device__ void run(double *p, double v) { atomicAdd(p, v); } };

template <> struct AtomicApply<int32_t, B200ALG_MAX> { static __device__ void run(int32_t *p, int32_t v) { atomicMax(p, v); } };
template <> struct AtomicApply<uint32_t, B200ALG_MAX> { static __device__ void run(uint32_t *p, uint32_t v) { atomicMax(p, v); } };
template <> struct AtomicApply<int64_t, B200ALG_MAX> { static __device__ void run(int64_t *p, int64_t v) { atomicMax((long long *)p, (long long)v); } };
template <> struct AtomicApply<uint64_t, B200ALG_MAX> { static __device__ void run(uint64_t *p, uint64_t v) { atomicMax((unsigned long long *)p, (unsigned long long)v); } };
template <> struct AtomicApply<int32_t, B200ALG_MIN> { static __device__ void run(int32_t *p, int32_t v) { atomicMin(p, v); } };
template <> struct AtomicApply<uint32_t, B200ALG_MIN> { static __device__ void run(uint32_t *p, uint32_t v) { atomicMin(p, v); } };
template <> struct AtomicApply<int64_t, B200ALG_MIN> { static __device__ void run(int64_t *p, int64_t v) { atomicMin((long long *)p, (long long)v); } };
template <> struct AtomicApply<uint64_t, B200ALG_MIN> { static __device__ void run(uint64_t *p, uint64_t v) { atomicMin((unsigned long long *)p, (unsigned long long)v); } };

// Float / double max and min: compare-and-swap on the bit pattern.
template <int OP> struct AtomicApply<float, OP> {
    static __device__ void run(float *p, float v) {
        unsigned int *u = (unsigned int *)p;
        unsigned int old = *u, assumed;
        do {
            assumed = old;
            float next = Op<float, OP>::apply(__uint_as_float(assumed), v);
            if (__float_as_uint(next) == assumed) break;
            old = atomicCAS(u, assumed, __float_as_uint(next));
        } while (old != assumed);
    }
};
template <int OP> struct AtomicApply<double, OP> {
    static __device__ void run(double *p, double v) {
        unsigned long long *u = (unsigned long long *)p;
        unsigned long long old = *u, assumed;
        do {
            assumed = old;
            double next = Op<double, OP>::apply(__longlong_as_double((long long)assumed), v);
            if ((unsigned long long)__double_as_longlong(next) == assumed) break;
            old = atomicCAS(u, assumed, (unsigned long long)__double_as_longlong(next));
        } while (old != assumed);
    }
};

// out[0] = Identity.  The reduction kernel is launched as a programmatic dependent of this
// one: its blocks fold their share of the input while this kernel runs and wait for it only
// before they combine into out[0].
template <typename T> __global__ void set_scalar_kernel(T *out, T v) {
    grid_dependency_release();
    *out = v;
}

template <typename T, int OP, int THREADS>
__device__ __forceinline__ void block_fold_and_publish(T acc, T *out) {
    using O = Op<T, OP>;
    __shared__ T warp_part[THREADS / 32];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc = O::apply(acc, shfl_down(acc, d));
    if (lane_id() == 0) warp_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        T v = threadIdx.x < THREADS / 32 ? warp_part[threadIdx.x] : O::identity();
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) v = O::apply(v, shfl_down(v, d));
        if (threadIdx.x == 0) {
            grid_dependency_wait();  // out[0] holds Identity from here on
            AtomicApply<T, OP>::run(out, v);
        }
    }
}

// Dense input.  The 16-byte aligned body is read as uint4 vectors with four loads in
// flight per thread; block 0 also folds the unaligned head and the tail.
template <typename T, int OP, int THREADS>
__global__ void __launch_bounds__(THREADS) reduce_dense_kernel(const T *__restrict__ in, int64_t n, T *out) {
    using O = Op<T, OP>;
    constexpr int VEC = 16 / sizeof(T);
    union V { uint4 u; T t[VEC]; };

    int64_t head = (int64_t)(((16u - (unsigned)((uintptr_t)in & 15u)) & 15u) / sizeof(T));
    if (head > n) head = n;
    const uint4 *vin = reinterpret_cast<const uint4 *>(in + head);
    const int64_t nvec = (n - head) / VEC;
    const int64_t tail = head + nvec * VEC;

    T acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = O::identity();

    const int64_t step = (int64_t)gridDim.x * THREADS;
    int64_t i = (int64_t)blockIdx.x * THREADS + threadIdx.x;
    for (; i + 3 * step < nvec; i += 4 * step) {
        V a, b, c, d;
        a.u = __ldcs(vin + i);
        b.u = __ldcs(vin + i + step);
        c.u = __ldcs(vin + i + 2 * step);
        d.u = __ldcs(vin + i + 3 * step);
#pragma unroll
        for (int k = 0; k < VEC; ++k)
            acc[k] = O::apply(O::apply(acc[k], a.t[k]), O::apply(b.t[k], O::apply(c.t[k], d.t[k])));
    }
    for (; i < nvec; i += step) {
        V a;
        a.u = __ldcs(vin + i);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = O::apply(acc[k], a.t[k]);
    }
    T r = acc[0];
#pragma unroll
    for (int k = 1; k < VEC; ++k) r = O::apply(r, acc[k]);
    if (blockIdx.x == 0) {
        for (int64_t j = threadIdx.x; j < head; j += THREADS) r = O::apply(r, in[j]);
        for (int64_t j = tail + threadIdx.x; j < n; j += THREADS) r = O::apply(r, in[j]);
    }
    block_fold_and_publish<T, OP, THREADS>(r, out);
}

// Stride1D.General input: element i lives at in[i * stride].
template <typename T, int OP, int THREADS>
__global__ void __launch_bounds__(THREADS) reduce_strided_kernel(const T *__restrict__ in, int64_t stride, int64_t n, T *out) {
    using O = Op<T, OP>;
    T r = O::identity();
    const int64_t step = (int64_t)gridDim.x * THREADS;
    for (int64_t i = (int64_t)blockIdx.x * THREADS + threadIdx.x; i < n; i += step) r = O::apply(r, in[i * stride]);
    block_fold_and_publish<T, OP, THREADS>(r, out);
}

template <typename T, int OP>
static int launch_reduce(cudaStream_t s, const void *in, int64_t stride, int64_t n, void *out) {
    constexpr int THREADS = 256;
    constexpr int VEC = 16 / sizeof(T);
    set_scalar_kernel<T><<<1, 1, 0, s>>>((T *)out, Op<T, OP>::identity());
    B200ALG_LAUNCH_CHECK();
    const int max_blocks = sm_count() * 8;
    if (stride == 1) {
        int64_t want = ceil_div(n, (int64_t)THREADS * VEC * 4);
        int blocks = (int)(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
        B200ALG_CUDA_TRY(launch_dependent(reduce_dense_kernel<T, OP, THREADS>, dim3(blocks), dim3(THREADS), 0, s, (const T *)in, n, (T *)out));
    } else {
        int64_t want = ceil_div(n, (int64_t)THREADS * 4);
        int blocks = (int)(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
        B200ALG_CUDA_TRY(launch_dependent(reduce_strided_kernel<T, OP, THREADS>, dim3(blocks), dim3(THREADS), 0, s, (const T *)in, stride, n, (T *)out));
    }
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

template <typename T>
static int dispatch_op(cudaStream_t s, const void *in, int64_t stride, int64_t n, int op, void *out) {
    switch (op) {
    case B200ALG_ADD: return launch_reduce<T, B200ALG_ADD>(s, in, stride, n, out);
    case B200ALG_MAX: return launch_reduce<T, B200ALG_MAX>(s, in, stride, n, out);
    case B200ALG_MIN: return launch_reduce<T, B200ALG_MIN>(s, in, stride, n, out);
    }
    return B200ALG_UNSUPPORTED;
}

}  // namespace b200alg

using namespace b200alg;

extern "C" int b200alg_reduce(void *stream, const void *in, int64_t stride, int64_t n, int dtype, int op, void *out) {
    // Argument checks keep the order of CreateReduction's (ReductionExtensions.cs:146-153).
    if (!in || !out) return B200ALG_INVALID_ARGUMENT;
    if (n < 1 || stride < 1) return B200ALG_INVALID_ARGUMENT;
    if (!is_atomic_numeric(dtype)) return B200ALG_UNSUPPORTED;
    const int es = dtype_bytes(dtype);
    if (((uintptr_t)in % es) || ((uintptr_t)out % es)) return B200ALG_MISALIGNED;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case B200ALG_I32: return dispatch_op<int32_t>(s, in, stride, n, op, out);
    case B200ALG_U32: return dispatch_op<uint32_t>(s, in, stride, n, op, out);
    case B200ALG_I64: return dispatch_op<int64_t>(s, in, stride, n, op, out);
    case B200ALG_U64: return dispatch_op<uint64_t>(s, in, stride, n, op, out);
    case B200ALG_F32: return dispatch_op<float>(s, in, stride, n, op, out);
    case B200ALG_F64: return dispatch_op<double>(s, in, stride, n, op, out);
    }
    return B200ALG_UNSUPPORTED;
}
