// Scan: single-pass chained scan with decoupled look-back.
// Replaces SinglePassScanKernel + its tile helpers (ScanExtensions.cs:284-388, :530-706),
// whose groups hand one running value down a strictly serial chain
// (SequentialGroupExecutor.cs:58-77) and read the input twice.  Here every tile is read
// once and written once (8 B / element for 4-byte types).
#include "common.cuh"
#include "lookback.cuh"

namespace b200alg {

constexpr int kScanThreads = 256;
constexpr int kScanWarps = kScanThreads / 32;
constexpr int kScanVecPerThread = 8;  // 8 x 16 bytes per thread -> 32 KB per tile

constexpr int kScanMinTileElems = 2 * kScanVecPerThread * kScanThreads;  // tile of an 8-byte type

// General variant (strided or unaligned views): one tile per block, handed out by an atomic
// ticket.  Thread t scans ITEMS consecutive elements of the tile, but global memory is touched
// warp-striped (consecutive lanes, consecutive elements: for a strided view, addresses one
// stride apart instead of ITEMS strides apart) and the warp transposes its chunk through
// shared memory, padded by one slot per 32 so that both access patterns are conflict-free.
template <typename T, int OP, bool INCLUSIVE>
__global__ void __launch_bounds__(kScanThreads)
scan_kernel(const T *in, int64_t in_stride, T *out, int64_t out_stride, int64_t n, const T *carry_in,
            TempHeader *hdr, void *state_base, int num_tiles) {
    using O = Op<T, OP>;
    constexpr int VEC = 16 / sizeof(T);
    constexpr int ITEMS = VEC * kScanVecPerThread;
    constexpr int TILE = ITEMS * kScanThreads;
    struct Items { T t[ITEMS]; };

    __shared__ T exchange[kScanWarps][32 * ITEMS + ITEMS];
    __shared__ T warp_total[kScanWarps];
    __shared__ T warp_excl[kScanWarps];
    __shared__ T s_prefix;
    __shared__ int s_tile;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    auto slot = [](int e) { return e + (e >> 5); };
    grid_dependency_wait();  // the descriptors and the ticket counter have been cleared
    if (tid == 0) s_tile = (int)atomicAdd(&hdr->reserved[0], 1u);
    __syncthreads();
    const int tile = s_tile;
    const int64_t base = (int64_t)tile * TILE;
    const int64_t remaining = n - base;

    Items it;
    const int64_t warp_first = (int64_t)warp * (32 * ITEMS);  // first element of the warp's chunk inside the tile
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
        const int e = j * 32 + lane;
        const int64_t idx = warp_first + e;
        exchange[warp][slot(e)] = idx < remaining ? in[(base + idx) * in_stride] : O::identity();
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) it.t[k] = exchange[warp][slot(lane * ITEMS + k)];

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

    __syncwarp();
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) exchange[warp][slot(lane * ITEMS + k)] = it.t[k];
    __syncwarp();
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
        const int e = j * 32 + lane;
        const int64_t idx = warp_first + e;
        if (idx < remaining) out[(base + idx) * out_stride] = exchange[warp][slot(e)];
    }
}

// Clears the control block and the tile descriptors a scan is about to use.  The scan kernel
// is launched as a programmatic dependent of this one, so its blocks are already resident
// (barriers initialised) when the last descriptor has been cleared.
__global__ void __launch_bounds__(256) scan_clear_kernel(uint4 *words, int64_t count) {
    grid_dependency_release();
    const int64_t step = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += step) words[i] = make_uint4(0u, 0u, 0u, 0u);
}

// ---- pipelined variant for dense, 16-byte aligned views ---------------------------------
// Persistent blocks take tiles round-robin (tile = blockIdx.x + k * gridDim.x).  A tile waits
// for the tiles before it, so every block of the grid has to be resident at the same time:
// the kernel is launched cooperatively, which makes the driver guarantee exactly that (or
// refuse the launch, in which case the ticketed kernel above runs instead).  Handing the
// tiles out by an atomic ticket, as the general kernel does, needs no such guarantee but
// measured 2.5 to 3 times slower on long inputs, whatever the prefetch distance.
// The input of the next tiles is staged into a shared-memory ring by bulk asynchronous
// copies (TMA, one elected thread, completion on an mbarrier), which keeps loads in flight
// while a block is busy with the scan and the look-back of its current tile.
constexpr int kScanStages = 2;
constexpr int kScanTileBytes = kScanThreads * kScanVecPerThread * 16;

template <typename T, int OP, bool INCLUSIVE>
__global__ void __launch_bounds__(kScanThreads)
scan_pipeline_kernel(const T *in, T *out, int64_t n, const T *carry_in, TempHeader *hdr, void *state_base, int num_tiles) {
    using O = Op<T, OP>;
    constexpr int VEC = 16 / sizeof(T);
    constexpr int NV = kScanVecPerThread;
    constexpr int TILE = VEC * NV * kScanThreads;
    union Vec { uint4 u; T t[VEC]; };

    extern __shared__ __align__(128) unsigned char ring[];  // kScanStages x kScanTileBytes
    __shared__ __align__(8) unsigned long long full_bar[kScanStages];
    __shared__ T warp_total[kScanWarps];
    __shared__ T warp_excl[kScanWarps];
    __shared__ T s_prefix;
    __shared__ int s_failed;               // a wait for a bulk copy ran out: later tiles are loaded directly

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int full_tiles = (int)(n / TILE);  // tiles below this index are complete

    // The last thread issues the copies: warp 0 does the look-back.
    constexpr int kStager = kScanThreads - 1;
    const int G = (int)gridDim.x;
    unsigned int in_flight = 0;  // stager: bit st set = a copy into stage st has not been waited for
    if (tid == kStager) {
        s_failed = 0;
        for (int st = 0; st < kScanStages; ++st) mbar_init(&full_bar[st], 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int st = 0; st < kScanStages; ++st) {
            const int t = (int)blockIdx.x + st * G;
            if (t < full_tiles) {
                mbar_expect_tx(&full_bar[st], kScanTileBytes);
                bulk_load(ring + st * kScanTileBytes, in + (int64_t)t * TILE, kScanTileBytes, &full_bar[st]);
                in_flight |= 1u << st;
            }
        }
    }
    __syncthreads();
    unsigned int bar_phase = 0;  // bit st = parity of the next completion of stage st's barrier
    bool staging = true;         // false once a wait for a copy ran out: later tiles are loaded directly
    TileState<T> state(state_base, num_tiles);

    int k = 0;
    for (int tile = (int)blockIdx.x; tile < num_tiles; tile += G, ++k) {
        const int st = k % kScanStages;
        const int64_t base = (int64_t)tile * TILE;
        const bool full = tile < full_tiles;
        const bool staged = full && staging;

        // Vector j of lane l covers elements (warp*32*NV + j*32 + l) * VEC ... + VEC of the tile.
        Vec v[NV];
        if (staged) {
            if (!mbar_wait(&full_bar[st], (bar_phase >> st) & 1u)) s_failed = 1;
            bar_phase ^= 1u << st;
            const uint4 *src = reinterpret_cast<const uint4 *>(ring + st * kScanTileBytes) + warp * (32 * NV);
#pragma unroll
            for (int j = 0; j < NV; ++j) v[j].u = src[j * 32 + lane];
            if (tid == kStager) in_flight &= ~(1u << st);
        } else {
#pragma unroll
            for (int j = 0; j < NV; ++j)
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const int64_t idx = base + (int64_t)(warp * (32 * NV) + j * 32 + lane) * VEC + e;
                    v[j].t[e] = idx < n ? in[idx] : O::identity();
                }
        }

        // inclusive scan inside each vector, then NV interleaved warp scans of the vector totals
        T w[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
#pragma unroll
            for (int e = 1; e < VEC; ++e) v[j].t[e] = O::apply(v[j].t[e - 1], v[j].t[e]);
            w[j] = v[j].t[VEC - 1];
        }
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const T up = shfl_up(w[j], d);
                if (lane >= d) w[j] = O::apply(up, w[j]);
            }
        }
        T before[NV];  // fold of everything in the warp's chunk that precedes vector j of this lane
        T chunk = O::identity();
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            T ex = shfl_up(w[j], 1);
            if (lane == 0) ex = O::identity();
            before[j] = O::apply(chunk, ex);
            chunk = O::apply(chunk, shfl_idx(w[j], 31));
        }
        if (lane == 31) warp_total[warp] = chunk;
        __syncthreads();  // warp totals are visible; every thread has taken its data out of the ring

        if (s_failed) staging = false;  // (read by every thread between the two barriers: uniform)
        if (tid == kStager && staging) {
            const int t2 = tile + kScanStages * G;
            if (t2 < full_tiles) {
                mbar_expect_tx(&full_bar[st], kScanTileBytes);
                bulk_load(ring + st * kScanTileBytes, in + (int64_t)t2 * TILE, kScanTileBytes, &full_bar[st]);
                in_flight |= 1u << st;
            }
        }

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

            T prefix;
            if (tile == 0) {
                prefix = carry_in ? *carry_in : O::identity();
                if (lane == 0) state.publish(0, kInclusive, O::apply(prefix, aggregate));
            } else {
                if (lane == 0) state.publish(tile, kAggregate, aggregate);
                // Decoupled look-back over kLookWays * 32 predecessors per round: lane l polls
                // the tiles at distances l+1, l+33, ... so that several loads are in flight per
                // lane; the operations are commutative, so the round's values are simply folded.
                constexpr int kLookWays = 1;
                constexpr int kLookLanes = 32;
                prefix = O::identity();
                int look = tile - 1 - lane;
                bool gave_up = false;
                while (true) {
                    T pv[kLookWays];
                    unsigned int flag[kLookWays];
#pragma unroll
                    for (int m = 0; m < kLookWays; ++m) {
                        pv[m] = O::identity();
                        flag[m] = kInclusive;  // tiles before tile 0 act as "inclusive identity"
                        if (lane >= kLookLanes) flag[m] = kAggregate;  // outside the window: contributes nothing
                        else if (look - 32 * m >= 0) flag[m] = state.poll(look - 32 * m, pv[m]);
                    }
#pragma unroll
                    for (int m = 0; m < kLookWays; ++m) {
                        unsigned int spins = 0;
                        while (flag[m] == kInvalid) {
                            if (++spins > kMaxSpin) { gave_up = true; flag[m] = kInclusive; pv[m] = O::identity(); break; }
                            __nanosleep(20);
                            flag[m] = state.poll(look - 32 * m, pv[m]);
                        }
                    }
                    // nearest predecessor with an inclusive prefix: smallest distance m*32 + lane
                    int nearest = kLookWays * 32;
#pragma unroll
                    for (int m = kLookWays - 1; m >= 0; --m) {
                        const unsigned int mask = __ballot_sync(0xffffffffu, flag[m] == kInclusive);
                        if (mask) nearest = m * 32 + (__ffs(mask) - 1);
                    }
                    T contrib = O::identity();
#pragma unroll
                    for (int m = 0; m < kLookWays; ++m)
                        if (m * 32 + lane <= nearest) contrib = O::apply(pv[m], contrib);
#pragma unroll
                    for (int d = 16; d > 0; d >>= 1) contrib = O::apply(shfl_down(contrib, d), contrib);
                    prefix = O::apply(shfl_idx(contrib, 0), prefix);
                    if (nearest < kLookWays * 32) break;
                    look -= kLookWays > 1 ? kLookWays * 32 : kLookLanes;
                }
                if (__any_sync(0xffffffffu, gave_up) && lane == 0) atomicExch(&hdr->wait_limit_hit, 1u);
                if (lane == 0) state.publish(tile, kInclusive, O::apply(prefix, aggregate));
            }
            if (lane == 0) s_prefix = prefix;
        }
        __syncthreads();

        const T warp_base = O::apply(s_prefix, warp_excl[warp]);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const T p = O::apply(warp_base, before[j]);
            if (INCLUSIVE) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) v[j].t[e] = O::apply(p, v[j].t[e]);
            } else {
#pragma unroll
                for (int e = VEC - 1; e > 0; --e) v[j].t[e] = O::apply(p, v[j].t[e - 1]);
                v[j].t[0] = p;
            }
        }
        if (full) {
            uint4 *dst = reinterpret_cast<uint4 *>(out + base) + warp * (32 * NV);
#pragma unroll
            for (int j = 0; j < NV; ++j) __stcs(dst + j * 32 + lane, v[j].u);
        } else {
#pragma unroll
            for (int j = 0; j < NV; ++j)
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const int64_t idx = base + (int64_t)(warp * (32 * NV) + j * 32 + lane) * VEC + e;
                    if (idx < n) out[idx] = v[j].t[e];
                }
        }
    }

    // A barrier wait that ran out is reported; copies that may still be in flight are given
    // one more bounded wait so that the block does not retire underneath them.
    __syncthreads();
    if (s_failed) {
        if (tid == kStager) {
            atomicExch(&hdr->wait_limit_hit, 1u);
            for (int st = 0; st < kScanStages; ++st)
                if (in_flight & (1u << st)) {
                    mbar_wait(&full_bar[st], 0u);
                    mbar_wait(&full_bar[st], 1u);
                }
        }
    }
}

template <typename T> constexpr int scan_tile_elems() { return (16 / (int)sizeof(T)) * kScanVecPerThread * kScanThreads; }

static int64_t scan_temp_bytes_for(int dtype, int64_t n) {
    // Sized for the smaller tile (8-byte types) so that one formula covers every type.
    const int64_t tiles = ceil_div(n < 1 ? 1 : n, kScanMinTileElems);
    (void)dtype;
    return (int64_t)sizeof(TempHeader) + round_up(tiles * kDescStride, 256);
}

template <typename T, int OP, bool INCLUSIVE>
static int launch_scan(cudaStream_t s, const void *in, int64_t in_stride, void *out, int64_t out_stride, int64_t n,
                       const void *carry_in, void *temp) {
    constexpr int TILE = scan_tile_elems<T>();
    const int64_t tiles64 = ceil_div(n, TILE);
    const int tiles = (int)tiles64;
    TempHeader *hdr = (TempHeader *)temp;
    void *state = (char *)temp + sizeof(TempHeader);
    const size_t state_bytes = (size_t)tiles * kDescStride;
    {
        const int64_t words = (int64_t)((sizeof(TempHeader) + state_bytes) / 16);
        const int64_t want = ceil_div(words, 256 * 4);
        const int64_t cap = (int64_t)sm_count() * 4;
        scan_clear_kernel<<<(int)(want < 1 ? 1 : (want > cap ? cap : want)), 256, 0, s>>>((uint4 *)temp, words);
        B200ALG_LAUNCH_CHECK();
    }
    const bool vec = in_stride == 1 && out_stride == 1 && ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0);
    bool launched = false;
    if (vec) {
        auto kernel = scan_pipeline_kernel<T, OP, INCLUSIVE>;
        constexpr size_t ring_bytes = (size_t)kScanStages * kScanTileBytes;
        static ContextCache<int> cache;  // per kernel instantiation and CUDA context
        int blocks_per_sm = 0;
        if (!cache.find(&blocks_per_sm)) {
            B200ALG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring_bytes));
            B200ALG_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, kernel, kScanThreads, ring_bytes));
            if (blocks_per_sm < 1) return B200ALG_UNSUPPORTED;
            cache.store(blocks_per_sm);
        }
        // One wave of persistent blocks, launched cooperatively: the driver either makes all of
        // them resident at once (tiles are taken round-robin and wait for one another) or
        // refuses the launch.
        const int resident = sm_count() * blocks_per_sm;
        const int blocks = tiles < resident ? tiles : resident;
        const T *in_t = (const T *)in;
        T *out_t = (T *)out;
        const T *carry_t = (const T *)carry_in;
        int64_t n_arg = n;
        int tiles_arg = tiles;
        void *args[] = {&in_t, &out_t, &n_arg, &carry_t, &hdr, &state, &tiles_arg};
        const cudaError_t e = cudaLaunchCooperativeKernel((const void *)kernel, dim3(blocks), dim3(kScanThreads), args, ring_bytes, s);
        if (e == cudaSuccess) launched = true;
        else if (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorNotSupported) (void)cudaGetLastError();
        else return cuda_fail(e);
    }
    if (!launched) {
        B200ALG_CUDA_TRY(launch_dependent(scan_kernel<T, OP, INCLUSIVE>, dim3(tiles), dim3(kScanThreads), 0, s, (const T *)in,
                                          in_stride, (T *)out, out_stride, n, (const T *)carry_in, hdr, state, tiles));
    }
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
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
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
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
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
constexpr size_t kStaticScanScratchBytes = sizeof(TempHeader) + (size_t)(kStaticScanMaxElements / kScanMinTileElems) * kDescStride;
static __device__ __align__(256) unsigned char g_static_scan_scratch[kStaticScanScratchBytes];

namespace b200alg {
// Device address of the array in the current CUDA context.  The array's name is only a handle
// on the host side, so the address is asked for once per context, with that context current.
int static_scan_scratch(void **out) {
    static ContextCache<void *> cache;
    void *p = nullptr;
    if (!cache.find(&p)) {
        B200ALG_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scan_scratch));
        cache.store(p);
    }
    *out = p;
    return B200ALG_OK;
}
}  // namespace b200alg

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
