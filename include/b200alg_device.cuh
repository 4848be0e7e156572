/*
 * b200alg - device-side building blocks for CUDA C++ kernels: block- and warp-wide radix sort
 * and permutation with the semantics of ILGPU.Algorithms' in-kernel helpers, plus the
 * element-wise transform / reorder launchers.  Header only; sm_100a (any sm_70+ compiles).
 *
 * Counterparts in the reference (Src/ILGPU.Algorithms):
 *   GroupRadixSort   GroupExtensions.RadixSort          GroupExtensions.cs:273-368
 *   WarpRadixSort    WarpExtensions.RadixSort           WarpExtensions.cs:97-130
 *   GroupPermute     GroupExtensions.Permute            GroupExtensions.cs:386-406
 *   WarpPermute      WarpExtensions.Permute             WarpExtensions.cs:147-166
 *   ComputeGroupWideRadixSortSharedMemorySize           RadixSortExtensions.cs:457-466
 *   Transform / Reorder / ReorderTransform              TransformExtensions.cs:377-506,
 *                                                        ReorderExtensions.cs:194-297
 * A C# kernel cannot call native device code, so these serve kernels written in CUDA C++
 * next to the library; results equal the reference's: a stable sort by the operation's
 * ExtractRadixBits order, one element per thread.
 */
#ifndef B200ALG_DEVICE_CUH
#define B200ALG_DEVICE_CUH

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200alg {
namespace device {

// ---- radix sort operations (IRadixSortOperation<T>, RadixSortOperations.tt:26-125) ---------
template <int BYTES> struct BitsOf;
template <> struct BitsOf<1> { using type = uint8_t; };
template <> struct BitsOf<2> { using type = uint16_t; };
template <> struct BitsOf<4> { using type = uint32_t; };
template <> struct BitsOf<8> { using type = uint64_t; };

enum class KeyKind { Unsigned, Signed, Floating, Half };
template <typename T> struct KeyKindOf { static constexpr KeyKind value = KeyKind::Unsigned; };
template <> struct KeyKindOf<int8_t> { static constexpr KeyKind value = KeyKind::Signed; };
template <> struct KeyKindOf<int16_t> { static constexpr KeyKind value = KeyKind::Signed; };
template <> struct KeyKindOf<int32_t> { static constexpr KeyKind value = KeyKind::Signed; };
template <> struct KeyKindOf<int64_t> { static constexpr KeyKind value = KeyKind::Signed; };
template <> struct KeyKindOf<float> { static constexpr KeyKind value = KeyKind::Floating; };
template <> struct KeyKindOf<double> { static constexpr KeyKind value = KeyKind::Floating; };
template <> struct KeyKindOf<__half> { static constexpr KeyKind value = KeyKind::Half; };

// Ascending{T} / Descending{T}.  Bits() is the value ExtractRadixBits shifts and masks:
// identity for unsigned keys, sign bit flipped for signed ones; for floating-point keys the
// reference's expression u ^ (signMask | (~u >> (NumBits - 1))) as written, where the shift
// is a logical one (Interop.FloatAsInt is unsigned), i.e. the sign bit is flipped and
// non-negative values also have their lowest bit flipped; Half: u ^ (0x8000 | ((uint)~u >> 15)).
template <typename T, bool DESCENDING> struct RadixSortOperation {
    using Bits = typename BitsOf<sizeof(T)>::type;
    static constexpr int NumBits = 8 * (int)sizeof(T);
    __host__ __device__ static T DefaultValue() { return T(); }
    __host__ __device__ static Bits RawBits(T v) {
        Bits u;
        memcpy(&u, &v, sizeof(T));
        return u;
    }
    __host__ __device__ static Bits KeyBits(T v) {
        const Bits u = RawBits(v);
        const Bits sign = (Bits)((Bits)1 << (NumBits - 1));
        Bits bits = u;
        if (KeyKindOf<T>::value == KeyKind::Signed) bits = u ^ sign;
        if (KeyKindOf<T>::value == KeyKind::Floating) bits = u ^ (sign | (Bits)((Bits)~u >> (NumBits - 1)));
        if (KeyKindOf<T>::value == KeyKind::Half) bits = (Bits)(u ^ (Bits)(0x8000u | ((uint32_t)~(uint32_t)u >> 15)));
        return DESCENDING ? (Bits)~bits : bits;
    }
    __host__ __device__ static int ExtractRadixBits(T v, int shift, int mask) { return (int)(KeyBits(v) >> shift) & mask; }
};
template <typename T> using Ascending = RadixSortOperation<T, false>;
template <typename T> using Descending = RadixSortOperation<T, true>;

// Shared memory a block of `group_size` threads needs for GroupRadixSort, in bytes: the
// reference's formula (elements, padding to ints, two arrays of warp-size ints, one int).
template <typename T> __host__ __device__ constexpr int ComputeGroupWideRadixSortSharedMemorySize(int group_size) {
    return (int)sizeof(T) * group_size + ((int)sizeof(T) * group_size) % 4 + 2 * 32 * 4 + 4;
}

namespace detail {
__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}
template <typename T> __device__ __forceinline__ T shuffle(T v, int lane) {
    static_assert(sizeof(T) <= 8, "element of at most 8 bytes");
    if constexpr (sizeof(T) == 8) {
        unsigned long long u;
        memcpy(&u, &v, 8);
        u = __shfl_sync(0xffffffffu, u, lane);
        memcpy(&v, &u, 8);
        return v;
    } else {
        unsigned int u = 0;
        memcpy(&u, &v, sizeof(T));
        u = __shfl_sync(0xffffffffu, u, lane);
        memcpy(&v, &u, sizeof(T));
        return v;
    }
}
}  // namespace detail

// ---- warp-wide sort: lane i receives the i-th element in the operation's order --------------
// One split per key bit: a vote tells every lane where the elements with a 0 bit and with a
// 1 bit go (stable), and every lane fetches the element that lands on it.  Call with all 32
// lanes.
template <typename T, typename TRadixSortOperation>
__device__ __forceinline__ T WarpRadixSort(T value) {
    const unsigned lane = threadIdx.x & 31u;
    for (int bit = 0; bit < TRadixSortOperation::NumBits; ++bit) {
        const bool one = TRadixSortOperation::ExtractRadixBits(value, bit, 1) != 0;
        const unsigned zeros_mask = __ballot_sync(0xffffffffu, !one);
        const unsigned zeros = __popc(zeros_mask);
        // the element that ends on this lane: the lane-th zero, or the (lane - zeros)-th one
        const int source = lane < zeros ? __fns(zeros_mask, 0, lane + 1) : __fns(~zeros_mask, 0, lane - zeros + 1);
        value = detail::shuffle(value, source);
    }
    return value;
}

// ---- block-wide sort: thread i receives the i-th element --------------------------------------
// One element per thread, 1-D block of a multiple of 32 threads (at most 1024), `shared`
// aligned to 8 bytes and of ComputeGroupWideRadixSortSharedMemorySize<T>(blockDim.x) bytes.
// One stable split per key bit: votes give the ranks inside each warp, the warps' counts of
// zeros and ones are chained through shared memory.
template <typename T, typename TRadixSortOperation>
__device__ __forceinline__ T GroupRadixSort(T value, unsigned char *shared) {
    const int dim = blockDim.x, i = threadIdx.x, lane = i & 31, warp = i >> 5, warps = dim >> 5;
    const int array_bytes = (int)sizeof(T) * dim;
    T *elements = reinterpret_cast<T *>(shared);
    int *zeros_before = reinterpret_cast<int *>(shared + array_bytes + array_bytes % 4);  // [32]: zeros in the warps before
    int *ones_before = zeros_before + 32;                                                  // [32]
    int *total_zeros = ones_before + 32;
    const unsigned lt = detail::lanemask_lt();
    elements[i] = value;
    __syncthreads();
    for (int bit = 0; bit < TRadixSortOperation::NumBits; ++bit) {
        const T element = elements[i];
        const bool one = TRadixSortOperation::ExtractRadixBits(element, bit, 1) != 0;
        const unsigned zeros_mask = __ballot_sync(0xffffffffu, !one);
        if (lane == 0) {
            zeros_before[warp] = __popc(zeros_mask);
            ones_before[warp] = 32 - __popc(zeros_mask);
        }
        __syncthreads();
        if (warp == 0) {  // exclusive scans of the two count arrays
            int z = lane < warps ? zeros_before[lane] : 0, o = lane < warps ? ones_before[lane] : 0;
            int zi = z, oi = o;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int zu = __shfl_up_sync(0xffffffffu, zi, d), ou = __shfl_up_sync(0xffffffffu, oi, d);
                if (lane >= d) { zi += zu; oi += ou; }
            }
            zeros_before[lane] = zi - z;
            ones_before[lane] = oi - o;
            if (lane == 31) *total_zeros = zi;
        }
        __syncthreads();
        const int target = one ? *total_zeros + ones_before[warp] + __popc(~zeros_mask & lt)
                               : zeros_before[warp] + __popc(zeros_mask & lt);
        __syncthreads();  // every thread has read its element and the counts
        elements[target] = element;
        __syncthreads();
    }
    return elements[i];
}

// ---- permutations ---------------------------------------------------------------------------
// The reference draws one random int per thread (rngView.Next()), keeps its upper bits, puts
// the thread index into the lower ones, sorts these keys and lets thread i take the element of
// the thread whose key came i-th.  `random` is that thread's draw; the same draws give the
// same permutation as the reference.
template <typename T> __device__ __forceinline__ T WarpPermute(T value, int random) {
    int key = (random & 0x7fffffc0) + (int)(threadIdx.x & 31u);
    key = WarpRadixSort<int, Ascending<int32_t>>(key);
    // lane i receives the element of lane (key & 0x3f): the reference scatters in a 32-step loop
    // (element of lane k goes to lane newLane[k]); the inverse gather below moves the same data
    const int new_lane = key & 0x3f;
    T result = T();
    for (int k = 0; k < 32; ++k) {
        const int target = __shfl_sync(0xffffffffu, new_lane, k);
        const T element = detail::shuffle(value, k);
        if (target == (int)(threadIdx.x & 31u)) result = element;
    }
    return result;
}

// shared: ComputeGroupWideRadixSortSharedMemorySize<T>(blockDim.x) rounded up to 8, followed by
// ComputeGroupWideRadixSortSharedMemorySize<int>(blockDim.x) bytes (the reference's layout:
// the element array, then the sort's memory).  Blocks of at most 1024 threads.
template <typename T> __device__ __forceinline__ T GroupPermute(T value, unsigned char *shared, int random) {
    const int dim = blockDim.x, i = threadIdx.x;
    const int array_bytes = (int)sizeof(T) * dim;
    T *elements = reinterpret_cast<T *>(shared);
    elements[i] = value;
    __syncthreads();
    int key = (random & 0x7ffffc00) + i;
    key = GroupRadixSort<int, Ascending<int32_t>>(key, shared + ((array_bytes + array_bytes % 4 + 7) & ~7));
    return elements[key & 0x3ff];
}

// ---- element-wise launchers -----------------------------------------------------------------
// Transformer: a functor with `TTarget operator()(TSource) const` (ITransformer<TSource, TTarget>).
template <typename TSource, typename TTarget, typename TTransformer>
__global__ void __launch_bounds__(256) transform_kernel(const TSource *source, int64_t source_stride, TTarget *target,
                                                        int64_t target_stride, int64_t n, TTransformer transformer) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        target[i * target_stride] = transformer(source[i * source_stride]);
}
template <typename TSource, typename TTarget, typename TIndex, typename TTransformer>
__global__ void __launch_bounds__(256) reorder_transform_kernel(const TSource *source, TTarget *target, const TIndex *reorder,
                                                                int64_t n, TTransformer transformer) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        target[i] = transformer(source[reorder[i]]);
}
struct IdentityTransformer {
    template <typename T> __host__ __device__ T operator()(T v) const { return v; }
};
namespace detail {
inline int grid_for(int64_t n) {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int64_t want = (n + 1023) / 1024, cap = (int64_t)sms * 8;
    return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}
}  // namespace detail

// target[i] = transformer(source[i])  (TransformExtensions.Transform; strides in elements)
template <typename TSource, typename TTarget, typename TTransformer>
inline cudaError_t Transform(cudaStream_t stream, const TSource *source, int64_t source_stride, TTarget *target,
                             int64_t target_stride, int64_t n, TTransformer transformer) {
    if (n <= 0) return cudaSuccess;
    transform_kernel<<<detail::grid_for(n), 256, 0, stream>>>(source, source_stride, target, target_stride, n, transformer);
    return cudaGetLastError();
}
// target[i] = transformer(source[reorder[i]])  (ReorderExtensions.ReorderTransform)
template <typename TSource, typename TTarget, typename TIndex, typename TTransformer>
inline cudaError_t ReorderTransform(cudaStream_t stream, const TSource *source, TTarget *target, const TIndex *reorder,
                                    int64_t n, TTransformer transformer) {
    if (n <= 0) return cudaSuccess;
    reorder_transform_kernel<<<detail::grid_for(n), 256, 0, stream>>>(source, target, reorder, n, transformer);
    return cudaGetLastError();
}
// target[i] = source[reorder[i]]  (ReorderExtensions.Reorder)
template <typename T, typename TIndex>
inline cudaError_t Reorder(cudaStream_t stream, const T *source, T *target, const TIndex *reorder, int64_t n) {
    return ReorderTransform(stream, source, target, reorder, n, IdentityTransformer());
}

}  // namespace device
}  // namespace b200alg
#endif /* B200ALG_DEVICE_CUH */
