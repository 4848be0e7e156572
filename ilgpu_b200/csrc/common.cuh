// Shared device/host helpers for the b200alg kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <float.h>
#include <limits.h>
#include <mutex>

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

// Number of SMs of the current device (148 on B200).
int sm_count();

// The CUDA context that is current on the calling thread, as an opaque handle (NULL when
// the driver cannot be asked).  A host such as ILGPU creates a context of its own per
// accelerator, so everything that CUDA keeps per context (function attributes, addresses of
// __device__ symbols) is cached by this handle, never by device ordinal.
void *current_context();

// Device address, in the current context, of the built-in scratch array of b200alg_scan_static.
int static_scan_scratch(void **out);

// A value per CUDA context, filled in on first use; safe for concurrent host threads.  A
// handful of contexts is the expected load, so the lookup is a linear scan under a mutex.
template <typename T> class ContextCache {
public:
    bool find(T *out) {
        void *ctx = current_context();
        if (!ctx) return false;
        std::lock_guard<std::mutex> g(mu_);
        for (int i = 0; i < used_; ++i)
            if (ctx_[i] == ctx) { *out = val_[i]; return true; }
        return false;
    }
    void store(const T &v) {
        void *ctx = current_context();
        if (!ctx) return;
        std::lock_guard<std::mutex> g(mu_);
        for (int i = 0; i < used_; ++i)
            if (ctx_[i] == ctx) { val_[i] = v; return; }
        if (used_ < kSlots) { ctx_[used_] = ctx; val_[used_] = v; ++used_; }
    }
private:
    static constexpr int kSlots = 64;
    std::mutex mu_;
    void *ctx_[kSlots] = {};
    T val_[kSlots] = {};
    int used_ = 0;
};

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

// Longest view an entry point accepts.  The reference stops at int.MaxValue elements
// (ErrorMessages.NotSupportedArrayView64); that check stays with the host-side mirror, the
// kernels index with 64 bits.
constexpr int64_t kMaxElements = 1ll << 38;  // per-block 32-bit counters of the histogram kernels hold up to here

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

// ---- bulk asynchronous copies (TMA) completing on an mbarrier -----------------------------
// Upper bound on polls of an mbarrier before a kernel gives up waiting for a bulk copy.
constexpr unsigned int kMaxBarrierPolls = 1u << 22;

__device__ __forceinline__ unsigned int smem_addr(const void *p) { return (unsigned int)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned int parity) {
    unsigned int ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bulk copy global -> this block's shared memory (no multicast); both addresses and the size
// are multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gsrc, unsigned int bytes, unsigned long long *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
// Bounded wait; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned int parity) {
    for (unsigned int polls = 0; polls < kMaxBarrierPolls; ++polls)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// ---- programmatic dependent launch ---------------------------------------------------------
// A kernel launched with launch_dependent() may start while the kernel before it on the
// stream still runs; it must call grid_dependency_wait() before it touches anything that
// kernel writes (the wait returns once the earlier kernel has completed and its writes are
// visible).  The earlier kernel calls grid_dependency_release() to let the next one start.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}

#endif  // __CUDACC__

}  // namespace b200alg
