// Scan: single-pass chained scan with decoupled look-back.
// Replaces SinglePassScanKernel + its tile helpers (ScanExtensions.cs:284-388, :530-706),
// whose groups hand one running value down a strictly serial chain
// (SequentialGroupExecutor.cs:58-77) and read the input twice.  Here every tile is read
// once and written once (8 B / element for 4-byte types).
#include "common.cuh"

namespace b200alg {

constexpr int kScanThreads = 256;
constexpr int kScanWarps = kScanThreads / 32;
constexpr int kScanVecPerThread = 4;  // 4 x 16 bytes per thread -> 16 KB per tile

enum : unsigned int { kInvalid = 0u, kAggregate = 1u, kInclusive = 2u };

// Tile descriptors.  4-byte types pack {flag, value} into one 64-bit word that is read
// and written with single (relaxed) accesses.  8-byte types keep the two partial results
// in separate slots and publish the flag with release / acquire.
template <typename T, int BYTES = sizeof(T)> struct TileState;

template <typename T> struct TileState<T, 4> {
    unsigned long long *words;
    __host__ __device__ TileState(void *base, int) : words((unsigned long long *)base) {}
    __device__ __forceinline__ void publish(int tile, unsigned int flag, T v) {
        unsigned int bits;
        memcpy(&bits, &v, 4);
        st_relaxed_u64(words + tile, ((unsigned long long)flag << 32) | bits);
    }
    __device__ __forceinline__ unsigned int poll(int tile, T &v) {
        unsigned long long w = ld_relaxed_u64(words + tile);
        unsigned int bits = (unsigned int)w;
        memcpy(&v, &bits, 4);
        return (unsigned int)(w >> 32);
    }
};

template <typename T> struct TileState<T, 8> {
    unsigned int *flags;
    T *agg;
    T *incl;
    __host__ __device__ TileState(void *base, int tiles) {
        agg = (T *)base;
        incl = agg + tiles;
        flags = (unsigned int *)(incl + tiles);
    }
    __device__ __forceinline__ void publish(int tile, unsigned int flag, T v) {
        T *slot = (flag == kInclusive ? incl : agg) + tile;
        unsigned long long bits;
        memcpy(&bits, &v, 8);
        st_relaxed_u64((unsigned long long *)slot, bits);
        st_release_u32(flags + tile, flag);
    }
    __device__ __forceinline__ unsigned int poll(int tile, T &v) {
        unsigned int f = ld_acquire_u32(flags + tile);
        if (f != kInvalid) {
            unsigned long long bits = ld_relaxed_u64((const unsigned long long *)((f == kInclusive ? incl : agg) + tile));
            memcpy(&v, &bits, 8);
        }
        return f;
    }
};

__device__ __forceinline__ int swz(int slot) { return slot ^ ((slot >> 3) & 7); }

template <typename T, int OP, bool INCLUSIVE, bool VECTOR>
__global__ void __launch_bounds__(kScanThreads)
scan_kernel(const T *in, int64_t in_stride, T *out, int64_t out_stride, int64_t n, const T *carry_in,
            TempHeader *hdr, void *state_base, int num_tiles) {
    using O = Op<T, OP>;
    constexpr int VEC = 16 / sizeof(T);
    constexpr int ITEMS = VEC * kScanVecPerThread;
    constexpr int TILE = ITEMS * kScanThreads;
    union Items { uint4 v[kScanVecPerThread]; T t[ITEMS]; };

    __shared__ uint4 xchg[kScanWarps][32 * kScanVecPerThread];
    __shared__ T warp_total[kScanWarps];
    __shared__ T warp_excl[kScanWarps];
    __shared__ T s_prefix;
    __shared__ int s_tile;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_tile = (int)atomicAdd(&hdr->reserved[0], 1u);
    __syncthreads();
    const int tile = s_tile;
    const int64_t base = (int64_t)tile * TILE;
    const int64_t remaining = n - base;
    const bool full = remaining >= TILE;

    Items it;
    if (VECTOR && full) {
        // Warp-striped 128-bit loads, then a warp-local transposition through swizzled
        // shared memory so that each thread holds ITEMS consecutive elements.
        const uint4 *src = reinterpret_cast<const uint4 *>(in + base) + warp * (32 * kScanVecPerThread);
#pragma unroll
        for (int j = 0; j < kScanVecPerThread; ++j) it.v[j] = __ldcs(src + j * 32 + lane);
#pragma unroll
        for (int j = 0; j < kScanVecPerThread; ++j) xchg[warp][swz(j * 32 + lane)] = it.v[j];
        __syncwarp();
#pragma unroll
        for (int j = 0; j < kScanVecPerThread; ++j) it.v[j] = xchg[warp][swz(lane * kScanVecPerThread + j)];
    } else {
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int64_t idx = (int64_t)tid * ITEMS + k;
            it.t[k] = idx < remaining ? in[(base + idx) * in_stride] : O::identity();
        }
    }

    // Thread total -> warp scan -> block scan.
    T tsum = it.t[0];
#pragma unroll
    for (int k = 1; k < ITEMS; ++k) tsum = O::apply(tsum, it.t[k]);
    T wincl = tsum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        T up = shfl_up(wincl, d);
        if (lane >= d) wincl = O::apply(up, wincl);
    }
    T lane_excl = shfl_up(wincl, 1);
    if (lane == 0) lane_excl = O::identity();
    if (lane == 31) warp_total[warp] = wincl;
    __syncthreads();

    if (warp == 0) {
        T wt = lane < kScanWarps ? warp_total[lane] : O::identity();
        T wi = wt;
#pragma unroll
        for (int d = 1; d < kScanWarps; d <<= 1) {
            T up = shfl_up(wi, d);
            if (lane >= d) wi = O::apply(up, wi);
        }
        T we = shfl_up(wi, 1);
        if (lane == 0) we = O::identity();
        if (lane < kScanWarps) warp_excl[lane] = we;
        const T aggregate = shfl_idx(wi, kScanWarps - 1);

        TileState<T> state(state_base, num_tiles);
        T prefix;
        if (tile == 0) {
            prefix = carry_in ? *carry_in : O::identity();
            if (lane == 0) state.publish(0, kInclusive, O::apply(prefix, aggregate));
        } else {
            if (lane == 0) state.publish(tile, kAggregate, aggregate);
            // Decoupled look-back: 32 predecessors per round, nearest first.
            prefix = O::identity();
            int look = tile - 1 - lane;
            bool gave_up = false;
            while (true) {
                T v = O::identity();
                unsigned int flag = kInclusive;  // tiles before tile 0 act as "inclusive identity"
                if (look >= 0) {
                    unsigned int spins = 0;
                    flag = state.poll(look, v);
                    while (flag == kInvalid) {
                        if (++spins > kMaxSpin) { gave_up = true; flag = kInclusive; v = O::identity(); break; }
                        __nanosleep(20);
                        flag = state.poll(look, v);
                    }
                }
                const unsigned int incl_mask = __ballot_sync(0xffffffffu, flag == kInclusive);
                // Lanes beyond the nearest tile with an inclusive prefix do not contribute.
                const int first = incl_mask ? (__ffs(incl_mask) - 1) : 31;
                T contrib = lane <= first ? v : O::identity();
                // In-order fold: lane 0 is the nearest predecessor, so fold from far to near.
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    T dn = shfl_down(contrib, d);
                    if (lane + d < 32) contrib = O::apply(dn, contrib);
                }
                const T window = shfl_idx(contrib, 0);
                prefix = O::apply(window, prefix);
                if (incl_mask) break;
                look -= 32;
            }
            if (__any_sync(0xffffffffu, gave_up) && lane == 0) atomicExch(&hdr->wait_limit_hit, 1u);
            if (lane == 0) state.publish(tile, kInclusive, O::apply(prefix, aggregate));
        }
        if (lane == 0) s_prefix = prefix;
    }
    __syncthreads();

    T running = O::apply(s_prefix, O::apply(warp_excl[warp], lane_excl));
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const T x = it.t[k];
        if (INCLUSIVE) {
            running = O::apply(running, x);
            it.t[k] = running;
        } else {
            it.t[k] = running;
            running = O::apply(running, x);
        }
    }

    if (VECTOR && full) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < kScanVecPerThread; ++j) xchg[warp][swz(lane * kScanVecPerThread + j)] = it.v[j];
        __syncwarp();
        uint4 *dst = reinterpret_cast<uint4 *>(out + base) + warp * (32 * kScanVecPerThread);
#pragma unroll
        for (int j = 0; j < kScanVecPerThread; ++j) __stcs(dst + j * 32 + lane, xchg[warp][swz(j * 32 + lane)]);
    } else {
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int64_t idx = (int64_t)tid * ITEMS + k;
            if (idx < remaining) out[(base + idx) * out_stride] = it.t[k];
        }
    }
}

template <typename T> constexpr int scan_tile_elems() { return (16 / (int)sizeof(T)) * kScanVecPerThread * kScanThreads; }

static int64_t scan_temp_bytes_for(int dtype, int64_t n) {
    // Sized for the smaller tile (8-byte types, 2048 elements) and the larger descriptor
    // (24 bytes per tile) so that one formula covers every type.
    const int64_t tiles = ceil_div(n < 1 ? 1 : n, 2048);
    (void)dtype;
    return (int64_t)sizeof(TempHeader) + round_up(tiles * 24, 256);
}

template <typename T, int OP, bool INCLUSIVE>
static int launch_scan(cudaStream_t s, const void *in, int64_t in_stride, void *out, int64_t out_stride, int64_t n,
                       const void *carry_in, void *temp) {
    constexpr int TILE = scan_tile_elems<T>();
    const int64_t tiles64 = ceil_div(n, TILE);
    const int tiles = (int)tiles64;
    TempHeader *hdr = (TempHeader *)temp;
    void *state = (char *)temp + sizeof(TempHeader);
    const size_t state_bytes = sizeof(T) == 4 ? (size_t)tiles * 8 : (size_t)tiles * 20;
    B200ALG_CUDA_TRY(cudaMemsetAsync(temp, 0, sizeof(TempHeader) + state_bytes, s));
    const bool vec = in_stride == 1 && out_stride == 1 && ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0);
    if (vec)
        scan_kernel<T, OP, INCLUSIVE, true><<<tiles, kScanThreads, 0, s>>>((const T *)in, 1, (T *)out, 1, n, (const T *)carry_in, hdr, state, tiles);
    else
        scan_kernel<T, OP, INCLUSIVE, false><<<tiles, kScanThreads, 0, s>>>((const T *)in, in_stride, (T *)out, out_stride, n, (const T *)carry_in, hdr, state, tiles);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

template <typename T, int OP>
static int dispatch_kind(cudaStream_t s, const void *in, int64_t is, void *out, int64_t os, int64_t n, int inclusive,
                         const void *carry, void *temp) {
    return inclusive ? launch_scan<T, OP, true>(s, in, is, out, os, n, carry, temp)
                     : launch_scan<T, OP, false>(s, in, is, out, os, n, carry, temp);
}

template <typename T>
static int dispatch_scan_op(cudaStream_t s, const void *in, int64_t is, void *out, int64_t os, int64_t n, int op,
                            int inclusive, const void *carry, void *temp) {
    switch (op) {
    case B200ALG_ADD: return dispatch_kind<T, B200ALG_ADD>(s, in, is, out, os, n, inclusive, carry, temp);
    case B200ALG_MAX: return dispatch_kind<T, B200ALG_MAX>(s, in, is, out, os, n, inclusive, carry, temp);
    case B200ALG_MIN: return dispatch_kind<T, B200ALG_MIN>(s, in, is, out, os, n, inclusive, carry, temp);
    }
    return B200ALG_UNSUPPORTED;
}

}  // namespace b200alg

using namespace b200alg;

extern "C" int b200alg_scan_temp_bytes(int dtype, int64_t n, int64_t *out_bytes) {
    if (!out_bytes || n < 0) return B200ALG_INVALID_ARGUMENT;
    if (!is_atomic_numeric(dtype)) return B200ALG_UNSUPPORTED;
    if (n > INT32_MAX) return B200ALG_TOO_LARGE;
    *out_bytes = scan_temp_bytes_for(dtype, n);
    return B200ALG_OK;
}

extern "C" int b200alg_scan_carry(void *stream, const void *in, int64_t in_stride, void *out, int64_t out_stride,
                                  int64_t n, int dtype, int op, int inclusive, const void *carry_in, void *temp,
                                  int64_t temp_bytes) {
    // Argument checks mirror CreateSinglePassScan's (ScanExtensions.cs:675-689).
    if (!in || !out || !temp) return B200ALG_INVALID_ARGUMENT;
    if (n < 0 || in_stride < 1 || out_stride < 1) return B200ALG_INVALID_ARGUMENT;
    if (!is_atomic_numeric(dtype)) return B200ALG_UNSUPPORTED;
    if (n > INT32_MAX) return B200ALG_TOO_LARGE;
    const int es = dtype_bytes(dtype);
    if (((uintptr_t)in % es) || ((uintptr_t)out % es) || (carry_in && ((uintptr_t)carry_in % es))) return B200ALG_MISALIGNED;
    if ((uintptr_t)temp % 256) return B200ALG_MISALIGNED;
    if (temp_bytes < scan_temp_bytes_for(dtype, n)) return B200ALG_TEMP_TOO_SMALL;
    if (n == 0) return B200ALG_OK;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case B200ALG_I32: return dispatch_scan_op<int32_t>(s, in, in_stride, out, out_stride, n, op, inclusive, carry_in, temp);
    case B200ALG_U32: return dispatch_scan_op<uint32_t>(s, in, in_stride, out, out_stride, n, op, inclusive, carry_in, temp);
    case B200ALG_I64: return dispatch_scan_op<int64_t>(s, in, in_stride, out, out_stride, n, op, inclusive, carry_in, temp);
    case B200ALG_U64: return dispatch_scan_op<uint64_t>(s, in, in_stride, out, out_stride, n, op, inclusive, carry_in, temp);
    case B200ALG_F32: return dispatch_scan_op<float>(s, in, in_stride, out, out_stride, n, op, inclusive, carry_in, temp);
    case B200ALG_F64: return dispatch_scan_op<double>(s, in, in_stride, out, out_stride, n, op, inclusive, carry_in, temp);
    }
    return B200ALG_UNSUPPORTED;
}

extern "C" int b200alg_scan(void *stream, const void *in, int64_t in_stride, void *out, int64_t out_stride, int64_t n,
                            int dtype, int op, int inclusive, void *temp, int64_t temp_bytes) {
    return b200alg_scan_carry(stream, in, in_stride, out, out_stride, n, dtype, op, inclusive, nullptr, temp, temp_bytes);
}

// ---- scan without caller-provided scratch ------------------------------------------------
// Some callers can neither size nor allocate a temp view: code that runs where device
// allocation is off the table (a host callback on a stream, a real-time loop that may not
// take the allocator's lock, a plug-in that is handed input and output views and nothing
// else).  For them the tile descriptors of the chained scan live in this fixed array,
// which every GPU that loads the library carries until the process exits.
constexpr int64_t kStaticScanMaxElements = 1ll << 26;
constexpr size_t kStaticScanScratchBytes = sizeof(TempHeader) + (size_t)(kStaticScanMaxElements / 2048) * 24;
static __device__ __align__(256) unsigned char g_static_scan_scratch[kStaticScanScratchBytes];

// Device address of the array on the current device.  The array's name is only a handle on
// the host side, so the address is asked for once per device, with that device current.
static int static_scan_scratch(void **out) {
    static void *address[64] = {nullptr};
    int dev = 0;
    B200ALG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B200ALG_UNSUPPORTED;
    if (address[dev] == nullptr) {
        void *p = nullptr;
        B200ALG_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scan_scratch));
        address[dev] = p;
    }
    *out = address[dev];
    return B200ALG_OK;
}

extern "C" int b200alg_scan_static(void *stream, const void *in, int64_t in_stride, void *out, int64_t out_stride,
                                   int64_t n, int dtype, int op, int inclusive) {
    if (n > kStaticScanMaxElements) return B200ALG_STATIC_LIMIT;
    void *scratch = nullptr;
    const int rc = static_scan_scratch(&scratch);
    if (rc != B200ALG_OK) return rc;
    // Same launch sequence as b200alg_scan: it clears the descriptors it is about to use, so
    // whatever the previous call left in the array does not matter.
    return b200alg_scan_carry(stream, in, in_stride, out, out_stride, n, dtype, op, inclusive, nullptr, scratch,
                              (int64_t)kStaticScanScratchBytes);
}
