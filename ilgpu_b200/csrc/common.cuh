// Shared device/host helpers for the b200alg kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <float.h>
#include <limits.h>

#include "../../include/b200alg.h"

namespace b200alg {

// ---- host side ------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return B200ALG_CUDA_ERROR;
}

#define B200ALG_CUDA_TRY(expr)                                   \
    do {                                                         \
        cudaError_t _e = (expr);                                 \
        if (_e != cudaSuccess) return ::b200alg::cuda_fail(_e);  \
    } while (0)

#define B200ALG_LAUNCH_CHECK() B200ALG_CUDA_TRY(cudaGetLastError())

// Number of SMs of the current device (148 on B200); cached per device ordinal.
int sm_count();

inline int dtype_bytes(int dt) {
    switch (dt) {
    case B200ALG_I8: case B200ALG_U8: return 1;
    case B200ALG_I16: case B200ALG_U16: case B200ALG_F16: return 2;
    case B200ALG_I32: case B200ALG_U32: case B200ALG_F32: return 4;
    case B200ALG_I64: case B200ALG_U64: case B200ALG_F64: return 8;
    }
    return 0;
}

inline bool is_atomic_numeric(int dt) {
    return dt == B200ALG_I32 || dt == B200ALG_U32 || dt == B200ALG_I64 || dt == B200ALG_U64 ||
           dt == B200ALG_F32 || dt == B200ALG_F64;
}

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Every temp buffer starts with this 256-byte control block.
struct TempHeader {
    unsigned int wait_limit_hit;   // set to 1 by a kernel whose bounded wait ran out
    unsigned int reserved[63];
};
static_assert(sizeof(TempHeader) == 256, "control block is 256 bytes");

// Upper bound on polls of one look-back slot before a kernel gives up (each poll is an
// L2 round trip of ~1 us under load, so this is seconds, far beyond any healthy run).
constexpr unsigned int kMaxSpin = 1u << 22;

// ---- device side ----------------------------------------------------------------------
#ifdef __CUDACC__

template <typename T> struct Limits;
template <> struct Limits<int32_t>  { static __host__ __device__ int32_t lowest() { return INT32_MIN; } static __host__ __device__ int32_t max() { return INT32_MAX; } };
template <> struct Limits<uint32_t> { static __host__ __device__ uint32_t lowest() { return 0u; } static __host__ __device__ uint32_t max() { return UINT32_MAX; } };
template <> struct Limits<int64_t>  { static __host__ __device__ int64_t lowest() { return INT64_MIN; } static __host__ __device__ int64_t max() { return INT64_MAX; } };
template <> struct Limits<uint64_t> { static __host__ __device__ uint64_t lowest() { return 0ull; } static __host__ __device__ uint64_t max() { return UINT64_MAX; } };
// C# float.MinValue / double.MinValue are -MaxValue, not -infinity.
template <> struct Limits<float>    { static __host__ __device__ float lowest() { return -FLT_MAX; } static __host__ __device__ float max() { return FLT_MAX; } };
template <> struct Limits<double>   { static __host__ __device__ double lowest() { return -DBL_MAX; } static __host__ __device__ double max() { return DBL_MAX; } };

// IScanReduceOperation<T> (IScanReduceOperation.cs:18-48) for Add / Max / Min.
template <typename T, int OP> struct Op;
template <typename T> struct Op<T, B200ALG_ADD> {
    static __host__ __device__ __forceinline__ T identity() { return T(0); }
    static __device__ __forceinline__ T apply(T a, T b) { return a + b; }
};
template <typename T> struct Op<T, B200ALG_MAX> {
    static __host__ __device__ __forceinline__ T identity() { return Limits<T>::lowest(); }
    static __device__ __forceinline__ T apply(T a, T b) { return a > b ? a : b; }
};
template <typename T> struct Op<T, B200ALG_MIN> {
    static __host__ __device__ __forceinline__ T identity() { return Limits<T>::max(); }
    static __device__ __forceinline__ T apply(T a, T b) { return a < b ? a : b; }
};
// Signed wrap-around like C# unchecked arithmetic.
template <> struct Op<int32_t, B200ALG_ADD> {
    static __host__ __device__ __forceinline__ int32_t identity() { return 0; }
    static __device__ __forceinline__ int32_t apply(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }
};
template <> struct Op<int64_t, B200ALG_ADD> {
    static __host__ __device__ __forceinline__ int64_t identity() { return 0; }
    static __device__ __forceinline__ int64_t apply(int64_t a, int64_t b) { return (int64_t)((uint64_t)a + (uint64_t)b); }
};

__device__ __forceinline__ unsigned lane_id() { return threadIdx.x & 31u; }
__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

template <typename T> __device__ __forceinline__ T shfl_up(T v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
template <typename T> __device__ __forceinline__ T shfl_down(T v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }
template <typename T> __device__ __forceinline__ T shfl_idx(T v, int l) { return __shfl_sync(0xffffffffu, v, l); }
template <> __device__ __forceinline__ int64_t shfl_up<int64_t>(int64_t v, int d) { return (int64_t)__shfl_up_sync(0xffffffffu, (long long)v, d); }
template <> __device__ __forceinline__ uint64_t shfl_up<uint64_t>(uint64_t v, int d) { return (uint64_t)__shfl_up_sync(0xffffffffu, (unsigned long long)v, d); }
template <> __device__ __forceinline__ int64_t shfl_down<int64_t>(int64_t v, int d) { return (int64_t)__shfl_down_sync(0xffffffffu, (long long)v, d); }
template <> __device__ __forceinline__ uint64_t shfl_down<uint64_t>(uint64_t v, int d) { return (uint64_t)__shfl_down_sync(0xffffffffu, (unsigned long long)v, d); }
template <> __device__ __forceinline__ int64_t shfl_idx<int64_t>(int64_t v, int l) { return (int64_t)__shfl_sync(0xffffffffu, (long long)v, l); }
template <> __device__ __forceinline__ uint64_t shfl_idx<uint64_t>(uint64_t v, int l) { return (uint64_t)__shfl_sync(0xffffffffu, (unsigned long long)v, l); }

// Memory-model helpers for the look-back protocols (gpu scope).
__device__ __forceinline__ void st_relaxed_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u32(unsigned int *p, unsigned int v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_relaxed_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_u32(unsigned int *p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

#endif  // __CUDACC__

}  // namespace b200alg
