// The library inside a CUDA context that is not the device's primary one - what ILGPU does:
// every CudaAccelerator creates a context of its own (Src/ILGPU/Runtime/Cuda/CudaAccelerator.cs:
// 170-175) and binds it before each call.  Function attributes, the opt-in to large shared
// memory and the address of the built-in scan scratch belong to a context, so the same calls
// run in the primary context, then in a second context on the same device, then in the first
// one again.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <numeric>
#include <random>
#include <vector>

#include "b200alg.h"

static int g_checks = 0, g_failures = 0;
#define CHECK(cond)                                                             \
    do {                                                                        \
        ++g_checks;                                                             \
        if (!(cond)) { ++g_failures; std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)

// One round of sort + scan + scan with built-in scratch in whatever context is current.
static void run_round(unsigned seed) {
    const int64_t n = 1000003;
    std::mt19937 rng(seed);
    std::vector<uint32_t> keys(n);
    for (auto &k : keys) k = rng();
    std::vector<int32_t> values(n);
    for (auto &v : values) v = (int32_t)(rng() % 100) - 50;

    uint32_t *dkeys = nullptr;
    int32_t *din = nullptr, *dout = nullptr, *dout2 = nullptr;
    void *temp = nullptr;
    int64_t sort_bytes = 0, scan_bytes = 0;
    CHECK(b200alg_radix_sort_temp_bytes(B200ALG_U32, n, 0, &sort_bytes) == B200ALG_OK);
    CHECK(b200alg_scan_temp_bytes(B200ALG_I32, n, &scan_bytes) == B200ALG_OK);
    CHECK(cudaMalloc(&dkeys, n * 4) == cudaSuccess);
    CHECK(cudaMalloc(&din, n * 4) == cudaSuccess);
    CHECK(cudaMalloc(&dout, n * 4) == cudaSuccess);
    CHECK(cudaMalloc(&dout2, n * 4) == cudaSuccess);
    CHECK(cudaMalloc(&temp, std::max(sort_bytes, scan_bytes)) == cudaSuccess);
    cudaMemcpy(dkeys, keys.data(), n * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(din, values.data(), n * 4, cudaMemcpyHostToDevice);

    CHECK(b200alg_radix_sort_keys(nullptr, dkeys, n, 1, B200ALG_U32, 0, temp, sort_bytes) == B200ALG_OK);
    CHECK(b200alg_device_status(nullptr, temp) == B200ALG_OK);
    std::vector<uint32_t> sorted(n);
    cudaMemcpy(sorted.data(), dkeys, n * 4, cudaMemcpyDeviceToHost);
    std::sort(keys.begin(), keys.end());
    CHECK(sorted == keys);

    CHECK(b200alg_scan(nullptr, din, 1, dout, 1, n, B200ALG_I32, B200ALG_ADD, 1, temp, scan_bytes) == B200ALG_OK);
    CHECK(b200alg_device_status(nullptr, temp) == B200ALG_OK);
    CHECK(b200alg_scan_static(nullptr, din, 1, dout2, 1, n, B200ALG_I32, B200ALG_ADD, 1) == B200ALG_OK);
    CHECK(b200alg_device_status(nullptr, nullptr) == B200ALG_OK);
    std::vector<int32_t> expect(n), got(n), got2(n);
    std::partial_sum(values.begin(), values.end(), expect.begin());
    cudaMemcpy(got.data(), dout, n * 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(got2.data(), dout2, n * 4, cudaMemcpyDeviceToHost);
    CHECK(got == expect);
    CHECK(got2 == expect);
    cudaFree(dkeys); cudaFree(din); cudaFree(dout); cudaFree(dout2); cudaFree(temp);
}

int main() {
    CHECK(cudaSetDevice(0) == cudaSuccess);
    CHECK(cudaFree(nullptr) == cudaSuccess);  // binds the primary context
    CUcontext primary = nullptr;
    CHECK(cuCtxGetCurrent(&primary) == CUDA_SUCCESS && primary != nullptr);
    run_round(1);

    CUdevice device;
    CHECK(cuDeviceGet(&device, 0) == CUDA_SUCCESS);
    CUcontext second = nullptr;
#if CUDA_VERSION >= 13000
    CHECK(cuCtxCreate(&second, nullptr, 0, device) == CUDA_SUCCESS);
#else
    CHECK(cuCtxCreate(&second, 0, device) == CUDA_SUCCESS);   // as CudaAccelerator does; becomes current
#endif
    CHECK(second != nullptr && second != primary);
    CHECK(cuCtxSetCurrent(second) == CUDA_SUCCESS);
    run_round(2);
    run_round(3);

    CHECK(cuCtxSetCurrent(primary) == CUDA_SUCCESS);
    run_round(4);
    CHECK(cuCtxSetCurrent(second) == CUDA_SUCCESS);
    run_round(5);
    CHECK(cuCtxSetCurrent(primary) == CUDA_SUCCESS);
    CHECK(cuCtxDestroy(second) == CUDA_SUCCESS);

    std::printf("contexts: %d checks, %d failures\n", g_checks, g_failures);
    return g_failures ? 1 : 0;
}
