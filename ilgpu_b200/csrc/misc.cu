// Library-wide helpers, status reporting, and the fill / iota kernels that sit on the
// edges of the path (InitializeExtensions.cs, SequenceExtensions.cs).
#include "common.cuh"

namespace b200alg {

thread_local int g_last_cuda_error = 0;

void *current_context() {
    // cuCtxGetCurrent through the runtime's table of driver entry points: no link-time
    // dependency on the driver library.
    typedef int (*GetCurrentFn)(void **);
    static GetCurrentFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (GetCurrentFn)p;
    }();
    void *ctx = nullptr;
    if (!fn || fn(&ctx) != 0) return nullptr;
    return ctx;  // NULL until the first runtime call of the thread has bound a context
}

int sm_count() {
    static ContextCache<int> cache;
    int v = 0;
    if (cache.find(&v)) return v;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
        return 148;
    cache.store(v);
    return v;
}

template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T *view, int64_t stride, int64_t n, T value) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) view[i * stride] = value;
}

template <typename T>
__global__ void __launch_bounds__(256) sequence_kernel(T *view, int64_t n, T start, T step_value) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        view[i] = (T)(start + (T)i * step_value);
}

// Test-only: one warp polls a word that nothing ever sets, with the same bounded-wait pattern
// as the look-back loops of the product kernels, and records that it gave up.
__global__ void wait_probe_kernel(TempHeader *hdr, const unsigned int *word, unsigned int max_polls) {
    unsigned int polls = 0;
    while (ld_acquire_u32(word) == 0u) {
        if (++polls > max_polls) {
            atomicExch(&hdr->wait_limit_hit, 1u);
            break;
        }
        __nanosleep(20);
    }
}

static int grid_for(int64_t n) {
    int64_t want = ceil_div(n, 256 * 4);
    int64_t cap = (int64_t)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace b200alg

using namespace b200alg;

extern "C" int b200alg_version(void) { return B200ALG_VERSION; }

extern "C" const char *b200alg_status_string(int status) {
    switch (status) {
    case B200ALG_OK: return "success";
    case B200ALG_INVALID_ARGUMENT: return "invalid argument";
    case B200ALG_UNSUPPORTED: return "unsupported element type, operation or value size";
    case B200ALG_TEMP_TOO_SMALL: return "temporary storage too small";
    case B200ALG_CUDA_ERROR: return "CUDA error (see b200alg_last_cuda_error)";
    case B200ALG_WAIT_LIMIT: return "a device-side wait exceeded its iteration limit";
    case B200ALG_MISALIGNED: return "pointer not aligned";
    case B200ALG_TOO_LARGE: return "more elements than the library indexes (2^38)";
    case B200ALG_STATIC_LIMIT: return "more elements than the built-in scratch of this entry point covers";
    case B200ALG_NCCL_ERROR: return "NCCL error (see b200alg_comm_last_nccl_error)";
    }
    return "unknown status";
}

extern "C" int b200alg_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int b200alg_initialize(void *stream, void *view, int64_t stride, int64_t n, int elem_bytes, const void *value) {
    if (n < 0 || stride < 1 || (n > 0 && !view) || !value) return B200ALG_INVALID_ARGUMENT;
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8 && elem_bytes != 16) return B200ALG_UNSUPPORTED;
    if (n == 0) return B200ALG_OK;
    if ((uintptr_t)view % elem_bytes) return B200ALG_MISALIGNED;
    cudaStream_t s = (cudaStream_t)stream;
    const int g = grid_for(n);
    switch (elem_bytes) {
    case 1: fill_kernel<uint8_t><<<g, 256, 0, s>>>((uint8_t *)view, stride, n, *(const uint8_t *)value); break;
    case 2: fill_kernel<uint16_t><<<g, 256, 0, s>>>((uint16_t *)view, stride, n, *(const uint16_t *)value); break;
    case 4: fill_kernel<uint32_t><<<g, 256, 0, s>>>((uint32_t *)view, stride, n, *(const uint32_t *)value); break;
    case 8: fill_kernel<uint64_t><<<g, 256, 0, s>>>((uint64_t *)view, stride, n, *(const uint64_t *)value); break;
    case 16: fill_kernel<uint4><<<g, 256, 0, s>>>((uint4 *)view, stride, n, *(const uint4 *)value); break;
    default: return B200ALG_UNSUPPORTED;
    }
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

extern "C" int b200alg_sequence(void *stream, void *view, int64_t n, int dtype, int64_t start, int64_t step) {
    if (n < 0 || (n > 0 && !view)) return B200ALG_INVALID_ARGUMENT;
    if (n == 0) return B200ALG_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int g = grid_for(n);
    switch (dtype) {
    case B200ALG_I32: case B200ALG_U32:
        if ((uintptr_t)view % 4) return B200ALG_MISALIGNED;
        sequence_kernel<uint32_t><<<g, 256, 0, s>>>((uint32_t *)view, n, (uint32_t)start, (uint32_t)step); break;
    case B200ALG_I64: case B200ALG_U64:
        if ((uintptr_t)view % 8) return B200ALG_MISALIGNED;
        sequence_kernel<uint64_t><<<g, 256, 0, s>>>((uint64_t *)view, n, (uint64_t)start, (uint64_t)step); break;
    default: return B200ALG_UNSUPPORTED;
    }
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

extern "C" int b200alg_testing_wait_limit(void *stream, void *temp, int64_t temp_bytes, unsigned int max_polls) {
    if (!temp || temp_bytes < 512 || ((uintptr_t)temp % 256)) return B200ALG_INVALID_ARGUMENT;
    if (max_polls > 1000000u) return B200ALG_INVALID_ARGUMENT;  // a test never waits long
    cudaStream_t s = (cudaStream_t)stream;
    B200ALG_CUDA_TRY(cudaMemsetAsync(temp, 0, 512, s));
    wait_probe_kernel<<<1, 32, 0, s>>>((TempHeader *)temp, (const unsigned int *)((const char *)temp + 256), max_polls);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

extern "C" int b200alg_device_status(void *stream, const void *temp) {
    if (!temp) {  // the built-in scratch array of b200alg_scan_static
        void *scratch = nullptr;
        const int rc = static_scan_scratch(&scratch);
        if (rc != B200ALG_OK) return rc;
        temp = scratch;
    }
    unsigned int flag = 0;
    cudaStream_t s = (cudaStream_t)stream;
    B200ALG_CUDA_TRY(cudaMemcpyAsync(&flag, temp, sizeof(flag), cudaMemcpyDeviceToHost, s));
    B200ALG_CUDA_TRY(cudaStreamSynchronize(s));
    return flag ? B200ALG_WAIT_LIMIT : B200ALG_OK;
}
