// Test program of include/b200alg_device.cuh: block- and warp-wide radix sort, permutations
// and the element-wise launchers, each against a host computation of what the reference's
// helpers yield (GroupExtensions.cs:273-406, WarpExtensions.cs:97-166, ReorderExtensions.cs,
// TransformExtensions.cs), and the key transforms against the CPU oracle.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <random>
#include <vector>

#include "b200alg_device.cuh"

extern "C" uint64_t oracle_key_bits(int dtype, uint64_t raw);  // oracle/ilgpu_cpu_oracle.c

using namespace b200alg::device;

static int g_checks = 0, g_failures = 0;
#define CHECK(cond)                                                             \
    do {                                                                        \
        ++g_checks;                                                             \
        if (!(cond)) { ++g_failures; std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)
#define CUDA_OK(expr)                                                           \
    do {                                                                        \
        cudaError_t e_ = (expr);                                                \
        if (e_ != cudaSuccess) { std::printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); return 2; } \
    } while (0)

template <typename T, typename Op> __global__ void group_sort_kernel(const T *in, T *out) {
    extern __shared__ __align__(8) unsigned char shared[];
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    out[i] = GroupRadixSort<T, Op>(in[i], shared);
}
template <typename T, typename Op> __global__ void warp_sort_kernel(const T *in, T *out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    out[i] = WarpRadixSort<T, Op>(in[i]);
}
template <typename T> __global__ void group_permute_kernel(const T *in, const int *random, T *out) {
    extern __shared__ __align__(8) unsigned char shared[];
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    out[i] = GroupPermute<T>(in[i], shared, random[i]);
}
template <typename T> __global__ void warp_permute_kernel(const T *in, const int *random, T *out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    out[i] = WarpPermute<T>(in[i], random[i]);
}

template <typename T> static std::vector<T> random_values(size_t n, unsigned seed, bool small_range) {
    std::mt19937_64 rng(seed);
    std::vector<T> v(n);
    for (auto &x : v) {
        uint64_t r = rng();
        if (small_range) r %= 7;   // many duplicates
        if (std::is_floating_point<T>::value) x = (T)((double)(int64_t)(r % 2001) - 1000.0) / (T)8;
        else x = (T)r;
    }
    return v;
}

template <typename T, typename Op> static std::vector<T> host_sorted(const std::vector<T> &v, size_t begin, size_t count) {
    std::vector<T> part(v.begin() + begin, v.begin() + begin + count);
    std::stable_sort(part.begin(), part.end(), [](const T &a, const T &b) { return Op::KeyBits(a) < Op::KeyBits(b); });
    return part;
}

template <typename T> static bool same_bits(const std::vector<T> &a, const std::vector<T> &b) {
    return a.size() == b.size() && std::memcmp(a.data(), b.data(), a.size() * sizeof(T)) == 0;
}

template <typename T, typename Op> static int sort_tests() {
    for (int block : {32, 64, 256, 1024}) {
        for (int variant = 0; variant < 2; ++variant) {
            const int blocks = 3;
            const size_t n = (size_t)block * blocks;
            auto host = random_values<T>(n, 17 * block + variant, variant == 1);
            T *in = nullptr, *out = nullptr;
            CUDA_OK(cudaMalloc(&in, n * sizeof(T)));
            CUDA_OK(cudaMalloc(&out, n * sizeof(T)));
            CUDA_OK(cudaMemcpy(in, host.data(), n * sizeof(T), cudaMemcpyHostToDevice));
            const int smem = (ComputeGroupWideRadixSortSharedMemorySize<T>(block) + 7) & ~7;
            group_sort_kernel<T, Op><<<blocks, block, smem>>>(in, out);
            std::vector<T> got(n);
            CUDA_OK(cudaMemcpy(got.data(), out, n * sizeof(T), cudaMemcpyDeviceToHost));
            for (int b = 0; b < blocks; ++b) {
                std::vector<T> part(got.begin() + (size_t)b * block, got.begin() + (size_t)(b + 1) * block);
                CHECK(same_bits(part, host_sorted<T, Op>(host, (size_t)b * block, block)));
            }
            warp_sort_kernel<T, Op><<<blocks, block>>>(in, out);
            CUDA_OK(cudaMemcpy(got.data(), out, n * sizeof(T), cudaMemcpyDeviceToHost));
            bool ok = true;
            for (size_t w = 0; w < n / 32; ++w) {
                std::vector<T> part(got.begin() + w * 32, got.begin() + (w + 1) * 32);
                ok = ok && same_bits(part, host_sorted<T, Op>(host, w * 32, 32));
            }
            CHECK(ok);
            cudaFree(in);
            cudaFree(out);
        }
    }
    return 0;
}

static int permute_tests() {
    for (int block : {32, 128, 1024}) {
        const int blocks = 2;
        const size_t n = (size_t)block * blocks;
        std::vector<int64_t> host(n);
        std::iota(host.begin(), host.end(), 1000);
        std::mt19937 rng(block);
        std::vector<int> random(n);
        for (auto &r : random) r = (int)(rng() & 0x7fffffff);
        int64_t *in = nullptr, *out = nullptr;
        int *drandom = nullptr;
        CUDA_OK(cudaMalloc(&in, n * 8));
        CUDA_OK(cudaMalloc(&out, n * 8));
        CUDA_OK(cudaMalloc(&drandom, n * 4));
        CUDA_OK(cudaMemcpy(in, host.data(), n * 8, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(drandom, random.data(), n * 4, cudaMemcpyHostToDevice));
        const int smem = ((ComputeGroupWideRadixSortSharedMemorySize<int64_t>(block) + 7) & ~7) +
                         ((ComputeGroupWideRadixSortSharedMemorySize<int>(block) + 7) & ~7);
        group_permute_kernel<int64_t><<<blocks, block, smem>>>(in, drandom, out);
        std::vector<int64_t> got(n);
        CUDA_OK(cudaMemcpy(got.data(), out, n * 8, cudaMemcpyDeviceToHost));
        for (int b = 0; b < blocks; ++b) {
            // thread i takes the element of the thread whose key (random bits above the index) came i-th
            std::vector<int> keys(block);
            for (int i = 0; i < block; ++i) keys[i] = (random[(size_t)b * block + i] & 0x7ffffc00) + i;
            std::vector<int> sorted = keys;
            std::sort(sorted.begin(), sorted.end());
            bool ok = true;
            for (int i = 0; i < block; ++i) ok = ok && got[(size_t)b * block + i] == host[(size_t)b * block + (sorted[i] & 0x3ff)];
            CHECK(ok);
            std::vector<int64_t> part(got.begin() + (size_t)b * block, got.begin() + (size_t)(b + 1) * block);
            std::sort(part.begin(), part.end());
            CHECK(std::equal(part.begin(), part.end(), host.begin() + (size_t)b * block));   // a permutation
        }
        warp_permute_kernel<int64_t><<<blocks, block>>>(in, drandom, out);
        CUDA_OK(cudaMemcpy(got.data(), out, n * 8, cudaMemcpyDeviceToHost));
        bool ok = true;
        for (size_t w = 0; w < n / 32; ++w) {
            std::vector<int> keys(32);
            for (int i = 0; i < 32; ++i) keys[i] = (random[w * 32 + i] & 0x7fffffc0) + i;
            std::vector<int> sorted = keys;
            std::sort(sorted.begin(), sorted.end());
            // the element of lane i goes to lane (sorted[i] & 0x3f)
            for (int i = 0; i < 32; ++i) ok = ok && got[w * 32 + (sorted[i] & 0x3f)] == host[w * 32 + i];
        }
        CHECK(ok);
        cudaFree(in);
        cudaFree(out);
        cudaFree(drandom);
    }
    return 0;
}

struct TimesThreePlusOne {
    __host__ __device__ double operator()(int v) const { return 3.0 * v + 1.0; }
};

static int launcher_tests() {
    const int64_t n = 100003;
    std::vector<int> host(n);
    std::iota(host.begin(), host.end(), -500);
    std::vector<int> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::shuffle(order.begin(), order.end(), std::mt19937(5));
    int *src = nullptr, *idx = nullptr, *same = nullptr;
    double *dst = nullptr;
    CUDA_OK(cudaMalloc(&src, n * 4));
    CUDA_OK(cudaMalloc(&idx, n * 4));
    CUDA_OK(cudaMalloc(&same, n * 4));
    CUDA_OK(cudaMalloc(&dst, 2 * n * 8));
    CUDA_OK(cudaMemcpy(src, host.data(), n * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(idx, order.data(), n * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemset(dst, 0, 2 * n * 8));
    CUDA_OK(Transform(nullptr, src, 1, dst, 2, n, TimesThreePlusOne()));      // strided target
    std::vector<double> got(2 * n);
    CUDA_OK(cudaMemcpy(got.data(), dst, 2 * n * 8, cudaMemcpyDeviceToHost));
    bool ok = true;
    for (int64_t i = 0; i < n; ++i) ok = ok && got[2 * i] == 3.0 * host[i] + 1.0 && got[2 * i + 1] == 0.0;
    CHECK(ok);
    CUDA_OK(Reorder(nullptr, src, same, idx, n));
    std::vector<int> moved(n);
    CUDA_OK(cudaMemcpy(moved.data(), same, n * 4, cudaMemcpyDeviceToHost));
    ok = true;
    for (int64_t i = 0; i < n; ++i) ok = ok && moved[i] == host[order[i]];
    CHECK(ok);
    CUDA_OK(ReorderTransform(nullptr, src, dst, idx, n, TimesThreePlusOne()));
    CUDA_OK(cudaMemcpy(got.data(), dst, n * 8, cudaMemcpyDeviceToHost));
    ok = true;
    for (int64_t i = 0; i < n; ++i) ok = ok && got[i] == 3.0 * host[order[i]] + 1.0;
    CHECK(ok);
    cudaFree(src); cudaFree(idx); cudaFree(same); cudaFree(dst);
    return 0;
}

template <typename T> static void key_bits_against_oracle(int dtype) {
    auto values = random_values<T>(2000, 99 + dtype, false);
    bool asc = true, desc = true;
    const uint64_t mask = sizeof(T) == 8 ? ~0ull : ((1ull << (8 * sizeof(T))) - 1);
    for (const T &v : values) {
        uint64_t raw = 0;
        std::memcpy(&raw, &v, sizeof(T));
        const uint64_t want = oracle_key_bits(dtype, raw) & mask;
        asc = asc && (uint64_t)Ascending<T>::KeyBits(v) == want;
        desc = desc && (uint64_t)Descending<T>::KeyBits(v) == ((~want) & mask);
    }
    CHECK(asc);
    CHECK(desc);
}

int main() {
    // dtype codes of include/b200alg.h
    key_bits_against_oracle<int8_t>(0); key_bits_against_oracle<uint8_t>(1); key_bits_against_oracle<int16_t>(2);
    key_bits_against_oracle<uint16_t>(3); key_bits_against_oracle<int32_t>(4); key_bits_against_oracle<uint32_t>(5);
    key_bits_against_oracle<int64_t>(6); key_bits_against_oracle<uint64_t>(7); key_bits_against_oracle<float>(9);
    key_bits_against_oracle<double>(10);
    int rc = 0;
    rc |= sort_tests<int32_t, Ascending<int32_t>>();
    rc |= sort_tests<int32_t, Descending<int32_t>>();
    rc |= sort_tests<uint32_t, Ascending<uint32_t>>();
    rc |= sort_tests<int64_t, Ascending<int64_t>>();
    rc |= sort_tests<uint64_t, Descending<uint64_t>>();
    rc |= sort_tests<float, Ascending<float>>();
    rc |= sort_tests<double, Descending<double>>();
    rc |= sort_tests<uint8_t, Ascending<uint8_t>>();
    rc |= sort_tests<int16_t, Ascending<int16_t>>();
    rc |= permute_tests();
    rc |= launcher_tests();
    if (rc) return rc;
    // the shared-memory size helper is the reference's formula
    CHECK(ComputeGroupWideRadixSortSharedMemorySize<int>(128) == 128 * 4 + 2 * 32 * 4 + 4);
    CHECK(ComputeGroupWideRadixSortSharedMemorySize<uint8_t>(33) == 33 + 1 + 2 * 32 * 4 + 4);
    std::printf("device header: %d checks, %d failures\n", g_checks, g_failures);
    return g_failures ? 1 : 0;
}
