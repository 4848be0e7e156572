// Radix sort: onesweep-style least-significant-digit sort with 8-bit digits.
//
//   1. one pass over the keys builds the histograms of ALL digit positions,
//   2. a one-block kernel turns them into global digit offsets and finds digit positions
//      on which every key agrees (those passes are skipped),
//   3. one kernel per remaining digit position: a tile of keys is ranked in shared memory
//      (the lanes of a warp meet in per-warp digit tables), the tile's digit counts are chained to the previous tiles'
//      with decoupled look-back, and the tile is scattered to its final place for that
//      digit - each key is read once and written once per pass.
//
// Replaces RadixSortKernel1 / RadixSortKernel2 and the host loop around them
// (RadixSortExtensions.cs:660-738, :852-912, :1276-1334: 2 bits per pass, 4 launches per
// pass) and, for pairs, the AoS gather / sort / scatter of :1047-1073 (values are carried
// structure-of-arrays here).  Every pass is a stable partition, so the result equals the
// reference's: a stable sort by the transformed key.
#include "common.cuh"

#include <type_traits>

namespace b200alg {

constexpr int kRadix = 256;
constexpr int kMaxPasses = 8;

// Control words that live in TempHeader::reserved.
enum : int {
    kCtlTicket = 0,        // [0..7]  next tile of each pass (tiles are handed out in order)
    kCtlSkip = 8,          // [8..15] 1 = every key has the same digit at this position
    kCtlSrc = 16,          // [16..23] buffer this pass reads (kBufIn / kBufOut / kBufAlt)
    kCtlFinal = 24,        // buffer the sorted data ended in (kBufOut: nothing left to do)
    kCtlFirstPass = 25,    // first pass that runs (kNoPass when every pass is skipped)
    kCtlDst = 32,          // [32..39] buffer this pass writes
    kCtlStatusHalf = 40    // [40..47] which of the two look-back arrays this pass uses
};
// The three buffers a sort moves its data between.
enum : unsigned int { kBufIn = 0, kBufOut = 1, kBufAlt = 2 };

// Views of one sort call.  An in-place sort has in == out (possibly strided); an out-of-place
// sort leaves `in` untouched.  The alternate buffer is dense scratch of n elements.
template <typename K, typename V> struct SortBuffers {
    const K *in;
    K *out, *alt;
    const V *vin;
    V *vout, *valt;
    int64_t stride;             // of the input / output view
    int64_t n;                  // element count, or its upper bound when n_device is set
    const long long *n_device;  // element count in device memory (NULL: n is exact)
};
template <typename K, typename V> __device__ __forceinline__ int64_t effective_n(const SortBuffers<K, V> &io) {
    if (!io.n_device) return io.n;
    const long long v = *io.n_device;
    return v < 0 ? 0 : (v > io.n ? io.n : (int64_t)v);
}
constexpr unsigned int kNoPass = 0xFFu;

// Values that are a function of the element's index (the reference's sequencers:
// IndexSequencer and the integer / Half / Float / Double sequencers, Sequencer.cs:37-72,
// Sequencers.tt:26-38): the pairs sort can produce them in its first pass instead of reading
// a value view.
enum : int { kSeqNone = 0, kSeqInteger = 1, kSeqFloating = 2 };
template <typename V> __device__ __forceinline__ V sequence_value(int kind, int64_t i) {
    if constexpr (sizeof(V) == 2) {
        if (kind == kSeqFloating) return (V)__half_as_ushort(__float2half_rn((float)i));
        return (V)i;
    } else if constexpr (sizeof(V) == 4) {
        if (kind == kSeqFloating) return (V)__float_as_uint((float)i);
        return (V)i;
    } else if constexpr (sizeof(V) == 8) {
        if (kind == kSeqFloating) return (V)__double_as_longlong((double)i);
        return (V)i;
    } else if constexpr (sizeof(V) == 1) {
        return (V)i;
    } else {
        return V{};
    }
}

// Key transform: bits = raw ^ (sign(raw) ? xor_neg : xor_pos) covers every key type of
// RadixSortOperations.tt:77-93 and the descending complement of :122-123.
template <typename K> struct KeyXform {
    K xor_neg, xor_pos;
    __device__ __forceinline__ K operator()(K raw) const {
        return raw ^ ((raw >> (sizeof(K) * 8 - 1)) ? xor_neg : xor_pos);
    }
};
// Ascending unsigned keys need no transform at all.
template <typename K> struct KeyIdentity {
    __device__ __forceinline__ K operator()(K raw) const { return raw; }
};

static bool key_xform_constants(int dtype, int order, uint64_t &xn, uint64_t &xp) {
    const int bits = dtype_bytes(dtype) * 8;
    const uint64_t all = bits == 64 ? ~0ull : ((1ull << bits) - 1);
    const uint64_t sign = 1ull << (bits - 1);
    const bool total = (order & B200ALG_SORT_FLOAT_TOTAL_ORDER) != 0;
    switch (dtype) {
    case B200ALG_U8: case B200ALG_U16: case B200ALG_U32: case B200ALG_U64: xn = 0; xp = 0; break;
    case B200ALG_I8: case B200ALG_I16: case B200ALG_I32: case B200ALG_I64: xn = sign; xp = sign; break;
    case B200ALG_F32: case B200ALG_F64:
        // literal reference transform: u ^ (signMask | (~u >> (bits-1))), logical shift
        if (total) { xn = all; xp = sign; } else { xn = sign; xp = sign | 1ull; }
        break;
    case B200ALG_F16:
        // literal: u ^ (0x8000 | ((uint)~u >> 15)), the shifted term is 0x1FFFE | !sign
        if (total) { xn = all; xp = sign; } else { xn = 0xFFFEull; xp = 0xFFFFull; }
        break;
    default: return false;
    }
    if (order & B200ALG_SORT_DESCENDING) { xn ^= all; xp ^= all; }
    return true;
}

// ---- 1. histograms of all digit positions ----------------------------------------------
constexpr int kHistoThreads = 1024;
// Counters per (digit position, digit): lane l uses replica l % replicas.  With 32 replicas
// every lane of a warp has a bank of its own and an atomic instruction is one wavefront
// whatever the digits are; that table (128 KB for 4-byte keys) takes one block per SM, so
// short inputs use 8 replicas and two blocks per SM instead.
constexpr int kHistoMaxSmem = 128 * 1024;

template <typename K, int RSHIFT>
__global__ void __launch_bounds__(kHistoThreads)
sort_histogram_kernel(const K *__restrict__ keys, int64_t stride, int64_t n, const long long *n_device, KeyXform<K> xf,
                      unsigned long long *ghist) {
    constexpr int P = sizeof(K);
    if (n_device) {
        const long long v = *n_device;
        n = v < 0 ? 0 : (v > n ? n : (int64_t)v);
    }
    constexpr int rshift = RSHIFT;
    // replicas are interleaved ([position][digit][replica]) so that the lanes of a warp spread
    // over the banks even when their digits collide
    extern __shared__ unsigned int sh[];  // P x 256 x replicas
    const int replicas = 1 << rshift;
    for (int i = threadIdx.x; i < replicas * P * kRadix; i += kHistoThreads) sh[i] = 0u;
    __syncthreads();
    unsigned int *mine = sh + (threadIdx.x & (replicas - 1));
    const int64_t step = (int64_t)gridDim.x * kHistoThreads;
    const int64_t gtid = (int64_t)blockIdx.x * kHistoThreads + threadIdx.x;
    auto count = [&](K raw) {
        const K b = xf(raw);
#pragma unroll
        for (int p = 0; p < P; ++p)
            atomicAdd(mine + ((p * kRadix + ((unsigned)(b >> (8 * p)) & 0xFFu)) << rshift), 1u);
    };
    if (stride == 1) {
        constexpr int VEC = 16 / sizeof(K);
        union V { uint4 u; K k[VEC]; };
        int64_t head = (int64_t)(((16u - (unsigned)((uintptr_t)keys & 15u)) & 15u) / sizeof(K));
        if (head > n) head = n;
        const uint4 *vin = reinterpret_cast<const uint4 *>(keys + head);
        const int64_t nvec = (n - head) / VEC;
        const int64_t tail = head + nvec * VEC;
        int64_t i = gtid;
        for (; i + step < nvec; i += 2 * step) {
            V a, b;
            a.u = __ldg(vin + i);
            b.u = __ldg(vin + i + step);
#pragma unroll
            for (int k = 0; k < VEC; ++k) count(a.k[k]);
#pragma unroll
            for (int k = 0; k < VEC; ++k) count(b.k[k]);
        }
        for (; i < nvec; i += step) {
            V a;
            a.u = __ldg(vin + i);
#pragma unroll
            for (int k = 0; k < VEC; ++k) count(a.k[k]);
        }
        if (blockIdx.x == 0) {
            for (int64_t j = threadIdx.x; j < head; j += kHistoThreads) count(keys[j]);
            for (int64_t j = tail + threadIdx.x; j < n; j += kHistoThreads) count(keys[j]);
        }
    } else {
        for (int64_t i = gtid; i < n; i += step) count(keys[i * stride]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < P * kRadix; i += kHistoThreads) {
        unsigned int c = 0;
        for (int r = 0; r < replicas; ++r) c += sh[(i << rshift) + ((r + threadIdx.x) & (replicas - 1))];
        if (c) atomicAdd(ghist + i, (unsigned long long)c);
    }
}

// ---- 2. global digit offsets, skipped passes, buffer schedule ---------------------------
// skip_enabled: a pass on whose digit every key agrees does not run.  out_of_place: the input
// view is only read; the passes then alternate between the output view and the alternate
// buffer so that the last one writes the output view.  In place, they alternate between the
// view and the alternate buffer, and the result is copied home if it ended in the latter.
__global__ void __launch_bounds__(kRadix)
sort_offsets_kernel(const unsigned long long *ghist, unsigned long long *gbase, TempHeader *hdr, int passes, long long n,
                    const long long *n_device, int skip_enabled, int out_of_place) {
    __shared__ unsigned long long warp_sum[kRadix / 32];
    __shared__ int s_skip;
    const int d = threadIdx.x, lane = d & 31, warp = d >> 5;
    if (n_device) {
        const long long v = *n_device;
        n = v < 0 ? 0 : (v > n ? n : v);
    }
    for (int p = 0; p < passes; ++p) {
        if (d == 0) s_skip = 0;
        __syncthreads();
        const unsigned long long c = ghist[p * kRadix + d];
        if (skip_enabled && c == (unsigned long long)n) s_skip = 1;
        unsigned long long incl = c;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1) {
            unsigned long long up = __shfl_up_sync(0xffffffffu, incl, k);
            if (lane >= k) incl += up;
        }
        if (lane == 31) warp_sum[warp] = incl;
        __syncthreads();
        unsigned long long before = 0;
        for (int w = 0; w < warp; ++w) before += warp_sum[w];
        gbase[p * kRadix + d] = before + incl - c;
        if (d == 0) hdr->reserved[kCtlSkip + p] = (unsigned)s_skip;
        __syncthreads();
    }
    if (d == 0) {
        int running = 0;
        for (int p = 0; p < passes; ++p) running += hdr->reserved[kCtlSkip + p] ? 0 : 1;
        unsigned int first = kNoPass, cur = out_of_place ? kBufIn : kBufOut;
        int j = 0;
        for (int p = 0; p < passes; ++p) {
            if (hdr->reserved[kCtlSkip + p]) continue;
            if (first == kNoPass) first = (unsigned)p;
            unsigned int dst;
            if (out_of_place) dst = ((running - 1 - j) & 1) ? kBufAlt : kBufOut;
            else dst = cur == kBufOut ? kBufAlt : kBufOut;
            hdr->reserved[kCtlSrc + p] = cur;
            hdr->reserved[kCtlDst + p] = dst;
            hdr->reserved[kCtlStatusHalf + p] = (unsigned)(j & 1);
            cur = dst;
            ++j;
        }
        hdr->reserved[kCtlFinal] = cur;
        hdr->reserved[kCtlFirstPass] = first;
    }
}

// ---- 3. one digit pass -------------------------------------------------------------------
// Look-back words: the top two bits carry the state, the rest the count.
template <typename SW> struct StatusWord;
template <> struct StatusWord<unsigned int> {
    static constexpr unsigned int kAgg = 1u << 30, kIncl = 2u << 30, kMask = (1u << 30) - 1u;
    static __device__ __forceinline__ void st(unsigned int *p, unsigned int v) { st_relaxed_u32(p, v); }
    static __device__ __forceinline__ unsigned int ld(const unsigned int *p) { return ld_relaxed_u32(p); }
};
template <> struct StatusWord<unsigned long long> {
    static constexpr unsigned long long kAgg = 1ull << 62, kIncl = 2ull << 62, kMask = (1ull << 62) - 1ull;
    static __device__ __forceinline__ void st(unsigned long long *p, unsigned long long v) { st_relaxed_u64(p, v); }
    static __device__ __forceinline__ unsigned long long ld(const unsigned long long *p) { return ld_relaxed_u64(p); }
};

// What a pass partitions by.  RadixDigit: one 8-bit digit of the transformed key.
// SplitterBucket: the number of splitters that are <= (key, global index) in the order
// (transformed key, index) - used to split a shard into per-rank buckets before the
// all-to-all of a multi-GPU sort; ties between equal keys are broken by position, which
// keeps the partition balanced under heavy duplicates and stable.
template <typename K, typename XF = KeyXform<K>> struct RadixDigit {
    static constexpr bool kUsesIndex = false;
    XF xf;
    int shift;
    __device__ __forceinline__ unsigned int operator()(K key, int64_t, const unsigned char *) const {
        return (unsigned int)(xf(key) >> shift) & 0xFFu;
    }
};
template <typename K> struct SplitterBucket {
    static constexpr bool kUsesIndex = true;
    static constexpr int kSmall = 7;  // up to this many splitters are compared without a loop
    // The tables a block keeps in shared memory (16-byte aligned), by byte offset: splitter
    // indices, transformed splitter keys, then (partition pass only) the destination pointers.
    // They are addressed from the block's shared-memory base, so the kernel holds no pointer to
    // them in registers.
    static constexpr int kIndexAt = 0, kKeysAt = kRadix * 8, kKeyPointersAt = kRadix * 16, kValuePointersAt = kRadix * 24;
    static constexpr int kTableBytes = kRadix * 32, kTableBytesWithoutPointers = kRadix * 16;
    KeyXform<K> xf;
    const K *splitter_keys;
    const int64_t *splitter_index;
    int num_splitters;
    int64_t index_base;
    // Optional: where each bucket of this shard goes (device arrays of num_splitters + 1
    // pointers; the targets may be peer-GPU memory mapped into this process).  When set, the
    // pass stores bucket b's elements at bucket_keys[b][0..count_b) instead of one output array.
    void *const *bucket_keys;
    void *const *bucket_values;

    // Fills the tables: keys already transformed, slots up to kSmall padded with the largest
    // key, which no key exceeds.  Call with all threads of the block, then synchronise.
    __device__ __forceinline__ void stage(unsigned char *tables, bool with_pointers) const {
        K *keys = reinterpret_cast<K *>(tables + kKeysAt);
        int64_t *index = reinterpret_cast<int64_t *>(tables + kIndexAt);
        for (int s = threadIdx.x; s < num_splitters; s += blockDim.x) {
            keys[s] = xf(splitter_keys[s]);
            index[s] = splitter_index[s];
        }
        for (int s = num_splitters + threadIdx.x; s < kSmall + 1; s += blockDim.x) keys[s] = (K) ~(K)0;
        if (with_pointers && bucket_keys) {
            void **kp = reinterpret_cast<void **>(tables + kKeyPointersAt);
            void **vp = reinterpret_cast<void **>(tables + kValuePointersAt);
            for (int s = threadIdx.x; s <= num_splitters; s += blockDim.x) {
                kp[s] = bucket_keys[s];
                if (bucket_values) vp[s] = bucket_values[s];
            }
        }
    }
    static __device__ __forceinline__ void *key_pointer(const unsigned char *tables, unsigned int bucket) {
        return reinterpret_cast<void *const *>(tables + kKeyPointersAt)[bucket];
    }
    static __device__ __forceinline__ void *value_pointer(const unsigned char *tables, unsigned int bucket) {
        return reinterpret_cast<void *const *>(tables + kValuePointersAt)[bucket];
    }
    // Up to SLOTS (1, 3 or 7) splitters, without a loop or a branch: the number of splitters with
    // a smaller key, and whether the next one has the same key (then resolve_tie decides).  The
    // slots come with 16-byte loads from one address for the whole warp.
    template <int SLOTS>
    __device__ __forceinline__ unsigned int few(K key, const unsigned char *tables, bool &tie) const {
        const K *sk = reinterpret_cast<const K *>(tables + kKeysAt);
        const K tk = xf(key);
        unsigned int b;
        if constexpr (SLOTS == 1) {
            const K only = sk[0];
            tie = only == tk;
            return only < tk;
        } else {
            // the slots ascend (unused ones hold the largest key): a search tree of selects
            constexpr int kVecs = ((SLOTS + 1) * (int)sizeof(K) + 15) / 16;
            union { uint4 v[kVecs]; K k[kVecs * 16 / sizeof(K)]; } s;
            const uint4 *from = reinterpret_cast<const uint4 *>(sk);
#pragma unroll
            for (int q = 0; q < kVecs; ++q) s.v[q] = from[q];
            if constexpr (SLOTS == 3) {
                const bool c1 = s.k[1] < tk;
                const bool c2 = (c1 ? s.k[2] : s.k[0]) < tk;
                b = (c1 ? 2u : 0u) + (c2 ? 1u : 0u);
            } else {
                const bool c1 = s.k[3] < tk;
                const bool c2 = (c1 ? s.k[5] : s.k[1]) < tk;
                const K upper = c2 ? s.k[6] : s.k[4], lower = c2 ? s.k[2] : s.k[0];
                const bool c3 = (c1 ? upper : lower) < tk;
                b = (c1 ? 4u : 0u) + (c2 ? 2u : 0u) + (c3 ? 1u : 0u);
            }
            tie = sk[b] == tk;  // slot b is the first that is not smaller (slot SLOTS is padding)
            return b;
        }
    }
    // b splitters have a smaller key than this element; walks over those with an equal key whose
    // index does not exceed the element's.
    // (Not inlined, and without `this`: the call sits in a branch that is almost never taken.)
    static __device__ __noinline__ unsigned int resolve_tie(KeyXform<K> xf, int64_t index_base, int num_splitters, K key,
                                                            int64_t local_index, const unsigned char *tables, unsigned int b) {
        const K *sk = reinterpret_cast<const K *>(tables + kKeysAt);
        const int64_t *si = reinterpret_cast<const int64_t *>(tables + kIndexAt);
        const K tk = xf(key);
        const int64_t gi = index_base + local_index;
        while ((int)b < num_splitters && sk[b] == tk && si[b] <= gi) ++b;
        return b;
    }
    // Any number of splitters (the partition uses few<> for up to kSmall of them): a linear count.
    __device__ __forceinline__ unsigned int operator()(K key, int64_t local_index, const unsigned char *tables) const {
        const K *sk = reinterpret_cast<const K *>(tables + kKeysAt);
        const K tk = xf(key);
        // The splitters ascend by (key, index): count those with a smaller key, then walk over
        // the (rare) ones with an equal key whose index does not exceed this element's.
        unsigned int b = 0;
        for (int j = 0; j < num_splitters; ++j) b += sk[j] < tk;
        if ((int)b < num_splitters && sk[b] == tk) {
            const int64_t *si = reinterpret_cast<const int64_t *>(tables + kIndexAt);
            const int64_t gi = index_base + local_index;
            while ((int)b < num_splitters && sk[b] == tk && si[b] <= gi) ++b;
        }
        return b;
    }
};

struct NoValue {};
template <typename V> struct ValueBytes { static constexpr int value = sizeof(V); };
template <> struct ValueBytes<NoValue> { static constexpr int value = 0; };

// Index of an element of the whole view: 32 bits while the look-back words are, else 64.
template <typename SW> struct IndexOf { using type = unsigned int; };
template <> struct IndexOf<unsigned long long> { using type = unsigned long long; };

// Full dense tiles are staged in shared memory by one bulk asynchronous copy (TMA, no
// multicast) that is issued a tile ahead.  (Measured against plain loads of the next tile into
// registers during the write-out: 1.22 ms against 1.31 ms for the 2^26-key sort.)
constexpr bool kSortTma = true;
constexpr int kLookWindow = 4;  // predecessors examined per look-back round (2 and 8 measured slower)
// The digit passes are launched as programmatic dependents of one another: the blocks of the
// next pass move in as those of this one leave and do their set-up before they wait for it.
constexpr bool kSortPdl = true;

template <typename K, typename V, bool KEEP_DIGITS, int THREADS, int ITEMS>
struct OnesweepSmem {
    static constexpr int TILE = THREADS * ITEMS;
    static constexpr int WARPS = THREADS / 32;
    static constexpr int VB = ValueBytes<V>::value;
    // keys and values are reordered side by side when that stays small enough for two blocks
    // per SM; otherwise the values reuse the keys' buffer in a second round
    static constexpr bool SPLIT = VB != 0 && (size_t)TILE * ((int)sizeof(K) + VB) <= 72 * 1024;
    static constexpr int SLOT = SPLIT ? (int)sizeof(K) + VB : ((int)sizeof(K) > VB ? (int)sizeof(K) : VB);
    // [sorted: the reorder buffer][counts per warp and digit][lane masks per warp and digit]
    // [digit's first slot in the tile, digit's count][digit's global offset][small words +
    // mbarrier][pass description][digit of every slot][splitters][staged keys]
    // The lane masks are only alive while a tile is ranked, the reorder buffer only afterwards:
    // when two blocks per SM would not fit otherwise, the masks live at the head of the
    // reorder buffer (and every warp clears its row again before it ranks the next tile).
    static constexpr size_t table_bytes = (size_t)WARPS * kRadix * 4;
    static constexpr size_t fixed_bytes = kRadix * 16 + 256 + (KEEP_DIGITS ? (size_t)TILE + kRadix * 32 : 0) + 128;
    static constexpr bool MASKS_IN_SORTED =
        (size_t)TILE * SLOT >= table_bytes &&
        (size_t)TILE * SLOT + 2 * table_bytes + fixed_bytes + (size_t)TILE * sizeof(K) > 112 * 1024;
    static constexpr size_t off_sorted = 0;
    static constexpr size_t off_count = (size_t)TILE * SLOT;
    static constexpr size_t off_mask = MASKS_IN_SORTED ? off_sorted : off_count + table_bytes;
    static constexpr size_t off_excl = off_count + table_bytes + (MASKS_IN_SORTED ? 0 : table_bytes);
    static constexpr size_t off_goff = off_excl + kRadix * 8;
    static constexpr size_t off_misc = off_goff + kRadix * 8;
    static constexpr size_t off_context = off_misc + 128;   // the block's PassContext
    static constexpr size_t off_digits = off_context + 128;
    static constexpr size_t off_splitters = off_digits + (KEEP_DIGITS ? (size_t)TILE : 0);
    // splitters: 256 positions (8 bytes), 256 keys (8 bytes), 2 x 256 destination pointers
    static constexpr size_t off_stage = (off_splitters + (KEEP_DIGITS ? (size_t)kRadix * 32 : 0) + 127) / 128 * 128;
    // The staging buffer of the bulk copies is dropped (keys are then loaded directly) where
    // it would cost the second block per SM.
    static constexpr size_t kTwoBlocksPerSm = 113 * 1024;
    static constexpr bool STAGED = kSortTma && (THREADS > 512 || off_stage + (size_t)TILE * sizeof(K) <= kTwoBlocksPerSm);
    static constexpr size_t bytes = off_stage + (STAGED ? (size_t)TILE * sizeof(K) : 0);
};

// Everything one block needs to know about the pass it works on.
template <typename K, typename V, typename SW> struct PassContext {
    const K *src;
    K *dst;
    int64_t src_stride, dst_stride;
    const V *vsrc;
    V *vdst;
    int64_t n;
    int num_tiles;
    bool dense;   // the source is contiguous
    bool bulk;    // full tiles of the source can be staged by bulk copies (dense, 16-byte aligned)
    int value_seq;  // not kSeqNone: this pass makes the values from the element index instead of reading them
    TempHeader *hdr;
    unsigned int *ticket;
    const unsigned long long *gbase;
    SW *status, *status_next;
};

// Hands out the block's next tile and, when that tile is a full one of a bulk-copyable
// source, starts the copy of its keys into the staging buffer.  One thread calls this once
// every thread of the block has taken the current tile's keys out of the staging buffer.
template <typename K, typename V, typename SW, int TILE, bool STAGED>
__device__ __forceinline__ int take_ticket(const PassContext<K, V, SW> &c, K *stage, unsigned long long *bar) {
    const int next = (int)atomicAdd(c.ticket, 1u);
    if (STAGED && c.bulk && next < c.num_tiles && (int64_t)(next + 1) * TILE <= c.n) {
        mbar_expect_tx(bar, (unsigned int)(TILE * sizeof(K)));
        bulk_load(stage, c.src + (int64_t)next * TILE, (unsigned int)(TILE * sizeof(K)), bar);
    }
    return next;
}

// One tile of one digit pass; returns the block's next tile.  FAST = the tile is full and both
// buffers are dense (no bounds checks, no stride arithmetic).  Keys are held in warp-striped
// order: item i of lane l is element warp * 32 * ITEMS + i * 32 + l of the tile.
template <typename K, typename V, typename SW, typename Digit, int THREADS, int ITEMS, bool FAST>
__device__ __forceinline__ int onesweep_tile(const PassContext<K, V, SW> &c, int tile, unsigned int &bulk_phase,
                                             K (&key)[ITEMS], bool &have_keys, const Digit &dg, unsigned char *smem_raw) {
    constexpr int WARPS = THREADS / 32;
    constexpr int TILE = THREADS * ITEMS;
    constexpr bool HAS_VALUES = ValueBytes<V>::value != 0;
    using S = StatusWord<SW>;
    using Idx = typename IndexOf<SW>::type;
    using L = OnesweepSmem<K, V, Digit::kUsesIndex, THREADS, ITEMS>;
    K *skeys = reinterpret_cast<K *>(smem_raw + L::off_sorted);
    V *svals = reinterpret_cast<V *>(smem_raw + L::off_sorted + (L::SPLIT ? (size_t)TILE * sizeof(K) : 0));
    // count_tbl[w][d]: number, later first slot, of the d-keys of warp w; mask_tbl[w][d]: lanes of
    // warp w that hold d in the item being ranked (zero between items)
    unsigned int *count_tbl = reinterpret_cast<unsigned int *>(smem_raw + L::off_count);
    unsigned int *mask_tbl = reinterpret_cast<unsigned int *>(smem_raw + L::off_mask);
    unsigned int *bin_excl = reinterpret_cast<unsigned int *>(smem_raw + L::off_excl);  // digit's first slot inside the tile
    unsigned int *bin_count = bin_excl + kRadix;                                         // digit's keys in the tile
    Idx *bin_goff = reinterpret_cast<Idx *>(smem_raw + L::off_goff);  // global index of slot p is bin_goff[d] + p
    unsigned int *misc = reinterpret_cast<unsigned int *>(smem_raw + L::off_misc);  // [0..7] sums of the digit warps, [8] next tile
    unsigned long long *bar = reinterpret_cast<unsigned long long *>(smem_raw + L::off_misc + 64);
    unsigned char *sdigit = smem_raw + L::off_digits;  // only when digits need the index
    K *stage = reinterpret_cast<K *>(smem_raw + L::off_stage);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t tile_base = (int64_t)tile * TILE;
    const int valid = FAST ? TILE : (int)((c.n - tile_base) < TILE ? (c.n - tile_base) : TILE);
    const int warp_base = warp * 32 * ITEMS + lane;
    unsigned int *my_count = count_tbl + warp * kRadix;
    unsigned int *my_mask = mask_tbl + warp * kRadix;

    // The warp's own row of the count table starts at zero (nobody else touches it before the
    // first block-wide barrier of the tile); its lane masks are left at zero by every item
    // unless they share their memory with the reorder buffer.
    {
        uint4 *zc = reinterpret_cast<uint4 *>(my_count), *zm = reinterpret_cast<uint4 *>(my_mask);
#pragma unroll
        for (int i = 0; i < kRadix / 4 / 32; ++i) {
            zc[i * 32 + lane] = make_uint4(0u, 0u, 0u, 0u);
            if (L::MASKS_IN_SORTED) zm[i * 32 + lane] = make_uint4(0u, 0u, 0u, 0u);  // the reorder buffer's leftovers
        }
    }

    // The tile's keys: out of the staging buffer, or already in registers (requested while the
    // block was finishing its previous tile), or loaded now.
    if (FAST && L::STAGED && c.bulk) {
        if (!mbar_wait(bar, bulk_phase) && lane == 0) atomicExch(&c.hdr->wait_limit_hit, 1u);
        bulk_phase ^= 1u;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) key[i] = stage[warp_base + i * 32];
    } else if (have_keys) {
    } else if (FAST) {
        const K *p = c.src + tile_base + warp_base;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) key[i] = p[i * 32];
    } else {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int64_t idx = tile_base + warp_base + i * 32;
            key[i] = idx < c.n ? c.src[idx * c.src_stride] : K(0);
        }
    }
    __syncwarp();

    // Ranking inside the warp: for every item, the lanes that hold the same digit have to find
    // each other.  Every lane ORs its bit into the digit's mask in the warp's table and reads
    // the mask back after a warp barrier; the lowest lane of the mask adds the number of its
    // lanes to the warp's count of that digit, clears the mask and hands the previous count to
    // the others.  (Finding the peers with one warp vote per digit bit costs no shared memory
    // but measured slower for any share of the items, and the hardware match instruction far
    // slower.)  After the loop the warp's table holds its digit counts.
    const unsigned int lt = lanemask_lt();
    const unsigned int my_bit = 1u << lane;
    const unsigned char *tables = smem_raw + L::off_splitters;  // of a SplitterBucket; unused otherwise
    unsigned int packed[ITEMS];  // (rank among the warp's keys of that digit) << 8 | digit
    // the lowest lane of `peers` adds their number to the warp's count of digit d; everybody gets
    // the count before and adds the peers in front of it
    auto take_ranks = [&](int i, unsigned int d, unsigned int peers, bool clear_mask) {
        unsigned int count = 0u;
        if ((peers & lt) == 0u) {  // lowest lane with this digit
            count = atomicAdd(&my_count[d], (unsigned int)__popc(peers));
            if (clear_mask) my_mask[d] = 0u;
        }
        __syncwarp();  // the counts advance item by item
        count = __shfl_sync(0xffffffffu, count, __ffs(peers) - 1);
        packed[i] = ((count + (unsigned int)__popc(peers & lt)) << 8) | d;
    };
    auto rank_by_tables = [&]() {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            unsigned int d;
            if (FAST) {
                d = dg(key[i], tile_base + warp_base + i * 32, tables);
            } else {
                const int local = warp_base + i * 32;
                d = local < valid ? dg(key[i], tile_base + local, tables) : 0xFFu;  // padding ranks behind every real key
            }
            atomicOr(&my_mask[d], my_bit);
            __syncwarp();
            const unsigned int peers = my_mask[d];
            __syncwarp();
            take_ranks(i, d, peers, true);
        }
    };
    if constexpr (Digit::kUsesIndex) {
        // A partition into up to eight buckets.  Buckets first, for all items, without a branch; an
        // element whose key equals a splitter's (rare) is settled by its index afterwards.  With
        // two or four buckets the tables would serialise (all lanes of a bucket hit one word), so
        // the lanes find their peers by warp votes on the bits the buckets differ in (and, in a
        // ragged tile, the bit that tells the padding digit from them); eight buckets spread over
        // the tables much as random digits do, and the votes would cost more issue slots.
        auto rank_few = [&](auto slots) {
            constexpr int SLOTS = decltype(slots)::value;
            constexpr int BITS = SLOTS == 1 ? 1 : 2;
            constexpr bool VOTES = SLOTS <= 3;  // eight buckets spread over the tables like digits do
            unsigned int ties = 0u;
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                bool tie;
                unsigned int d = dg.template few<SLOTS>(key[i], tables, tie);
                if (!FAST && warp_base + i * 32 >= valid) {
                    d = 0xFFu;
                    tie = false;
                }
                packed[i] = d;
                ties |= tie ? 1u << i : 0u;
            }
            if (ties) {
#pragma unroll
                for (int i = 0; i < ITEMS; ++i)
                    if ((ties >> i) & 1u)
                        packed[i] = Digit::resolve_tie(dg.xf, dg.index_base, dg.num_splitters, key[i], tile_base + warp_base + i * 32,
                                                       tables, packed[i]);
            }
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const unsigned int d = packed[i];
                unsigned int peers;
                if constexpr (VOTES) {
                    peers = 0xffffffffu;
#pragma unroll
                    for (int b = 0; b < BITS + (FAST ? 0 : 1); ++b) {
                        const bool bit = ((d >> (b < BITS ? b : 3)) & 1u) != 0u;
                        const unsigned int m = __ballot_sync(0xffffffffu, bit);
                        peers &= bit ? m : ~m;
                    }
                } else {
                    atomicOr(&my_mask[d], my_bit);
                    __syncwarp();
                    peers = my_mask[d];
                    __syncwarp();
                }
                take_ranks(i, d, peers, !VOTES);
            }
        };
        const int ns = dg.num_splitters;  // uniform over the grid
        if (ns <= 1) rank_few(std::integral_constant<int, 1>{});
        else if (ns <= 3) rank_few(std::integral_constant<int, 3>{});
        else if (ns <= Digit::kSmall) rank_few(std::integral_constant<int, 7>{});
        else rank_by_tables();
    } else {
        rank_by_tables();
    }
    __syncthreads();  // A: the tables are complete; every thread has its keys out of the staging buffer

    // The values are not held during the ranking: sixteen more live registers there spill.
    V val[HAS_VALUES ? ITEMS : 1];
    if constexpr (HAS_VALUES) {  // requested now, in flight while the digit threads work, needed for the reorder
        bool from_index = false;
        if constexpr (sizeof(V) <= 8) from_index = c.value_seq != kSeqNone;
        if (from_index) {
            if constexpr (sizeof(V) <= 8) {
#pragma unroll
                for (int i = 0; i < ITEMS; ++i) val[i] = sequence_value<V>(c.value_seq, tile_base + warp_base + i * 32);
            }
        } else {
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const int local = warp_base + i * 32;
                if (FAST || local < valid) val[i] = c.vsrc[tile_base + local];
            }
        }
    }

    if (tid == THREADS - 1) misc[8] = (unsigned int)take_ticket<K, V, SW, TILE, L::STAGED>(c, stage, bar);

    // The first 256 threads (one per digit) turn the warps' digit counts into slots of the
    // reorder buffer and publish the tile's counts for the tiles behind it.
    if (tid < kRadix) {
        c.status_next[(size_t)tile * kRadix + tid] = 0;
        // entry [w][d] becomes the number of d-keys in the warps before w
        unsigned int run = 0;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const unsigned int cnt = count_tbl[w * kRadix + tid];
            count_tbl[w * kRadix + tid] = run;
            run += cnt;
        }
        const unsigned int tile_count = run;
        S::st(c.status + (size_t)tile * kRadix + tid, (tile == 0 ? S::kIncl : S::kAgg) | (SW)tile_count);
        bin_count[tid] = tile_count;
        // exclusive scan of the digit counts over the 256 digit threads
        unsigned int incl = tile_count;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1) {
            unsigned int up = __shfl_up_sync(0xffffffffu, incl, k);
            if (lane >= k) incl += up;
        }
        if (lane == 31) misc[warp] = incl;
        asm volatile("bar.sync 1, %0;" ::"n"(kRadix) : "memory");  // the digit threads among themselves
        unsigned int before = 0;
#pragma unroll
        for (int w = 0; w < kRadix / 32; ++w) before += (w < warp) ? misc[w] : 0u;
        const unsigned int excl = incl - tile_count + before;
        bin_excl[tid] = excl;
        // fold the digit's first slot into the per-warp offsets: one table lookup per key
#pragma unroll
        for (int w = 0; w < WARPS; ++w) count_tbl[w * kRadix + tid] += excl;
    }
    __syncthreads();  // C: every key has its slot

    // Reorder through shared memory so that global writes run along digit segments.
    constexpr bool SECOND_ROUND = HAS_VALUES && !L::SPLIT;  // the values follow through the same buffer
    unsigned int pos[SECOND_ROUND ? ITEMS : 1];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const unsigned int d = packed[i] & 0xFFu;
        const unsigned int slot = (packed[i] >> 8) + my_count[d];
        skeys[slot] = key[i];
        if constexpr (Digit::kUsesIndex) {
            if (dg.num_splitters > Digit::kSmall) sdigit[slot] = (unsigned char)d;  // few buckets: found again from the slot
        }
        if constexpr (L::SPLIT) svals[slot] = val[i];
        if constexpr (SECOND_ROUND) pos[i] = slot;
    }
    // The key registers are free again.  Unless the next tile arrives through the staging
    // buffer, request its keys now: the loads are in flight during the look-back and the
    // write-out.
    {
        const int next = (int)misc[8];
        const bool next_full = (int64_t)(next + 1) * TILE <= c.n;
        have_keys = false;
        if (next < c.num_tiles && !(L::STAGED && c.bulk && next_full)) {
            const int64_t next_base = (int64_t)next * TILE;
            if (c.dense && next_full) {
                const K *p = c.src + next_base + warp_base;
#pragma unroll
                for (int i = 0; i < ITEMS; ++i) key[i] = p[i * 32];
            } else {
#pragma unroll
                for (int i = 0; i < ITEMS; ++i) {
                    const int64_t idx = next_base + warp_base + i * 32;
                    key[i] = idx < c.n ? c.src[idx * c.src_stride] : K(0);
                }
            }
            have_keys = true;
        }
    }
    // Decoupled look-back by the last 256 threads, one digit per thread, kLookWindow
    // predecessors per round (their loads are independent, so a round costs one trip to L2).
    // It comes after the reorder: started earlier, beside the offset phases, it only walked
    // further back and polled more, and the pass got slower.
    constexpr int kWalkers = THREADS - kRadix;  // first thread of the look-back group
    if (tid >= kWalkers) {
        const int dgt = tid - kWalkers;
        Idx prefix = 0;
        if (tile > 0) {
            bool gave_up = false, done = false;
            int t = tile - 1;
            while (!done) {
                SW window[kLookWindow];
#pragma unroll
                for (int k = 0; k < kLookWindow; ++k)
                    window[k] = t - k >= 0 ? S::ld(c.status + (size_t)(t - k) * kRadix + dgt) : (SW)S::kIncl;
#pragma unroll
                for (int k = 0; k < kLookWindow; ++k) {
                    if (!done) {
                        SW w = window[k];
                        unsigned int spins = 0;
                        while ((w & ~S::kMask) == 0) {
                            if (++spins > kMaxSpin) { gave_up = true; break; }
                            __nanosleep(20);
                            w = S::ld(c.status + (size_t)(t - k) * kRadix + dgt);
                        }
                        if (gave_up) {
                            done = true;
                        } else {
                            prefix += (Idx)(w & S::kMask);
                            if (w & S::kIncl) done = true;
                        }
                    }
                }
                t -= kLookWindow;
            }
            if (gave_up) atomicExch(&c.hdr->wait_limit_hit, 1u);
            S::st(c.status + (size_t)tile * kRadix + dgt, S::kIncl | (SW)(prefix + bin_count[dgt]));
        }
        bin_goff[dgt] = (Idx)c.gbase[dgt] + prefix - (Idx)bin_excl[dgt];
    }
    __syncthreads();  // D

    // With few buckets (the ranks of one box) the write-out goes bucket by bucket: a bucket is a
    // run of consecutive slots with one destination, so nothing is looked up per element.
    bool few_buckets = false;
    if constexpr (Digit::kUsesIndex) few_buckets = dg.num_splitters <= Digit::kSmall;
    auto store_runs = [&](bool keys_too, bool values_too) {
        if constexpr (Digit::kUsesIndex) {
            const bool scattered = dg.bucket_keys != nullptr;
            // A run is stored so that every warp writes whole, aligned 128-byte lines of the
            // destination (the first lanes take the elements in front of the first line start):
            // stores into a peer's memory are not merged on the way, a line written in two pieces
            // crosses NVLink as two packets.
            auto store_run = [&](auto *dest, const auto *from, int lo, int hi, Idx g) {
                using T = std::remove_const_t<std::remove_reference_t<decltype(*dest)>>;
                if (hi <= lo) return;
                T *to = dest + (Idx)(g + (Idx)lo);                             // where the run's first element goes
                const int past = (int)(((uintptr_t)to / sizeof(T)) & 31u);     // its distance from a warp-sized line start
                to -= past;                                                    // slot v of the run's lines: to[v] = run[v - past]
                const T *run = from + lo - past;
                const int end = past + (hi - lo);
                for (int v = tid; v < end; v += THREADS)
                    if (v >= past) to[v] = run[v];
            };
            for (int b = 0; b <= dg.num_splitters; ++b) {
                const int lo = (int)bin_excl[b], hi = (int)bin_excl[b + 1];  // padding keys rank last
                const Idx g = bin_goff[b];  // modulo 2^32 or 2^64: only g + p is an index
                if (keys_too) {
                    K *kd = scattered ? reinterpret_cast<K *>(Digit::key_pointer(tables, b)) : c.dst;
                    if (scattered || FAST) {
                        store_run(kd, skeys, lo, hi, g);
                    } else {
                        for (int p = lo + tid; p < hi; p += THREADS) kd[(int64_t)(Idx)(g + (Idx)p) * c.dst_stride] = skeys[p];
                    }
                }
                if constexpr (!std::is_same<V, NoValue>::value) {
                    if (values_too) {
                        V *vd = scattered && dg.bucket_values ? reinterpret_cast<V *>(Digit::value_pointer(tables, b)) : c.vdst;
                        store_run(vd, svals, lo, hi, g);
                    }
                }
            }
        }
    };
    Idx out_idx[SECOND_ROUND ? ITEMS : 1];
    if (few_buckets) {
        store_runs(true, L::SPLIT);
    } else {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int p = tid + i * THREADS;
            if (FAST || p < valid) {
                const K k = skeys[p];
                unsigned int d;
                if constexpr (Digit::kUsesIndex) d = sdigit[p]; else d = dg(k, 0, tables);
                const Idx at = bin_goff[d] + (Idx)p;
                if constexpr (SECOND_ROUND) out_idx[i] = at;
                bool stored = false;
                if constexpr (Digit::kUsesIndex) {
                    if (dg.bucket_keys) {  // plain stores, possibly over NVLink into a peer's receive buffer
                        reinterpret_cast<K *>(Digit::key_pointer(tables, d))[at] = k;
                        stored = true;
                    }
                }
                if (!stored) {
                    if (FAST) c.dst[at] = k; else c.dst[(int64_t)at * c.dst_stride] = k;
                }
                if constexpr (L::SPLIT) {  // the value travels with its key
                    bool vstored = false;
                    if constexpr (Digit::kUsesIndex) {
                        if (dg.bucket_values) {
                            reinterpret_cast<V *>(Digit::value_pointer(tables, d))[at] = svals[p];
                            vstored = true;
                        }
                    }
                    if (!vstored) c.vdst[at] = svals[p];
                }
            }
        }
    }

    if constexpr (SECOND_ROUND) {
        __syncthreads();  // every key has left the reorder buffer
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int local = warp_base + i * 32;
            if (FAST || local < valid) svals[pos[i]] = val[i];
        }
        __syncthreads();
        if (few_buckets) {
            store_runs(false, true);
        } else {
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const int p = tid + i * THREADS;
                if (FAST || p < valid) {
                    bool stored = false;
                    if constexpr (Digit::kUsesIndex) {
                        if (dg.bucket_values) {
                            reinterpret_cast<V *>(Digit::value_pointer(tables, sdigit[p]))[out_idx[i]] = svals[p];
                            stored = true;
                        }
                    }
                    if (!stored) c.vdst[out_idx[i]] = svals[p];
                }
            }
        }
    }
    const int next_tile = (int)misc[8];
    __syncthreads();  // E: the reorder buffer and the tables are reused by the block's next tile
    return next_tile;
}

// Persistent blocks.  Tiles are handed out by an atomic ticket, in order, so a tile only ever
// waits for tiles whose blocks already run: forward progress does not depend on how many
// blocks of the grid are resident.
template <typename K, typename V, typename SW, typename Digit, int THREADS, int ITEMS>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS)
onesweep_kernel(SortBuffers<K, V> io, int pass, Digit dg, TempHeader *hdr, const unsigned long long *gbase_all,
                SW *status_all, int max_tiles, int value_seq) {
    constexpr int TILE = THREADS * ITEMS;
    static_assert(THREADS >= 2 * kRadix, "one thread per digit for the offsets and one for the look-back");
    using L = OnesweepSmem<K, V, Digit::kUsesIndex, THREADS, ITEMS>;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    if (kSortPdl) grid_dependency_release();  // the next kernel of the call may take the SMs this one leaves
    {   // The part of the set-up that reads nothing: the lane masks of the ranking tables start at
        // zero and are left at zero by every item.
        uint4 *zm = reinterpret_cast<uint4 *>(smem_raw + L::off_mask);
        for (int i = threadIdx.x; i < (THREADS / 32) * kRadix / 4; i += THREADS) zm[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    if (kSortPdl) grid_dependency_wait();  // everything the kernels before this one wrote is visible from here on
    if (hdr->reserved[kCtlSkip + pass]) return;
    // The pass description lives in shared memory: a dozen pointers that would otherwise sit
    // in registers for the whole kernel.
    static_assert(sizeof(PassContext<K, V, SW>) <= 128, "context slot");
    PassContext<K, V, SW> &c = *reinterpret_cast<PassContext<K, V, SW> *>(smem_raw + L::off_context);
    unsigned int *misc = reinterpret_cast<unsigned int *>(smem_raw + L::off_misc);
    const int64_t n = effective_n(io);
    const int num_tiles = (int)((n + TILE - 1) / TILE);
    if (threadIdx.x == THREADS - 1) {
        const unsigned int src = hdr->reserved[kCtlSrc + pass], dst = hdr->reserved[kCtlDst + pass];
        c.src = src == kBufIn ? io.in : (src == kBufOut ? io.out : io.alt);
        c.dst = dst == kBufOut ? io.out : io.alt;
        c.src_stride = src == kBufAlt ? 1 : io.stride;
        c.dst_stride = dst == kBufAlt ? 1 : io.stride;
        c.vsrc = src == kBufIn ? io.vin : (src == kBufOut ? io.vout : io.valt);
        c.vdst = dst == kBufOut ? io.vout : io.valt;
        c.n = n;
        c.num_tiles = num_tiles;
        c.dense = io.stride == 1;
        c.bulk = c.dense && ((uintptr_t)c.src % 16 == 0);
        c.value_seq = hdr->reserved[kCtlFirstPass] == (unsigned int)pass ? value_seq : kSeqNone;
        c.hdr = hdr;
        c.ticket = &hdr->reserved[kCtlTicket + pass];
        c.gbase = gbase_all + pass * kRadix;
        // Two look-back arrays alternate between the passes that run; this pass clears the
        // slots the next one will use (the previous pass, their last user, has completed).
        const bool upper = hdr->reserved[kCtlStatusHalf + pass] != 0;
        c.status = status_all + (upper ? (size_t)max_tiles * kRadix : 0);
        c.status_next = status_all + (upper ? 0 : (size_t)max_tiles * kRadix);
        unsigned long long *bar = reinterpret_cast<unsigned long long *>(smem_raw + L::off_misc + 64);
        if (L::STAGED) {
            mbar_init(bar, 1u);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        misc[8] = (unsigned int)take_ticket<K, V, SW, TILE, L::STAGED>(c, reinterpret_cast<K *>(smem_raw + L::off_stage), bar);
    }
    if constexpr (Digit::kUsesIndex)
        dg.stage(smem_raw + L::off_splitters, true);
    __syncthreads();
    int tile = (int)misc[8];
    __syncthreads();  // misc[8] is written again during the first tile
    const bool dense = io.stride == 1;
    unsigned int bulk_phase = 0u;
    K key[ITEMS];
    bool have_keys = false;
    while (tile < num_tiles) {
        if (dense && (int64_t)(tile + 1) * TILE <= n)
            tile = onesweep_tile<K, V, SW, Digit, THREADS, ITEMS, true>(c, tile, bulk_phase, key, have_keys, dg, smem_raw);
        else
            tile = onesweep_tile<K, V, SW, Digit, THREADS, ITEMS, false>(c, tile, bulk_phase, key, have_keys, dg, smem_raw);
    }
}

// ---- 4. bring the result home when it did not end in the output view ---------------------
template <typename K, typename V>
__global__ void __launch_bounds__(256)
sort_copy_back_kernel(SortBuffers<K, V> io, const TempHeader *hdr, int value_seq) {
    const int64_t n = effective_n(io);
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned int final_in = hdr->reserved[kCtlFinal];
    bool values_made = false;
    if constexpr (ValueBytes<V>::value != 0 && sizeof(V) <= 8) {
        // no pass ran (every key equal): the keys stay in order, the values still have to be made
        if (value_seq != kSeqNone && hdr->reserved[kCtlFirstPass] == kNoPass) {
            for (int64_t i = first; i < n; i += step) io.vout[i] = sequence_value<V>(value_seq, i);
            values_made = true;
        }
    }
    if (final_in == kBufOut) return;
    if (final_in == kBufIn && (const void *)io.in == (const void *)io.out) return;
    const K *from = final_in == kBufAlt ? io.alt : io.in;
    const V *vfrom = final_in == kBufAlt ? io.valt : io.vin;
    const int64_t from_stride = final_in == kBufAlt ? 1 : io.stride;
    for (int64_t i = first; i < n; i += step) {
        io.out[i * io.stride] = from[i * from_stride];
        if constexpr (ValueBytes<V>::value != 0) {
            if (!values_made) io.vout[i] = vfrom[i];
        }
    }
}

// ---- host side ---------------------------------------------------------------------------
struct SortLayout {
    int passes;
    int tile;
    int64_t tiles;
    bool wide_status;
    int64_t off_ghist, off_gbase, off_status, control_bytes, off_keys, off_values, total;
};

// Block shape of the digit pass: 512 threads, two blocks per SM, 8192 keys per tile (4096 for
// 8-byte keys).  256- and 1024-thread blocks, 12 and 24 items per thread all measured slower.
constexpr int kSortThreads = 512;
constexpr int kSortItems = 16;
template <typename K> struct SortTuning {
    static constexpr int THREADS = kSortThreads;
    static constexpr int ITEMS = sizeof(K) == 8 ? kSortItems / 2 : kSortItems;
};

static SortLayout sort_layout(int key_bytes, int value_bytes, int64_t n) {
    SortLayout L;
    L.passes = key_bytes;
    L.tile = kSortThreads * (key_bytes == 8 ? kSortItems / 2 : kSortItems);
    L.tiles = ceil_div(n < 1 ? 1 : n, L.tile);
    L.wide_status = n >= (1ll << 30);
    L.off_ghist = sizeof(TempHeader);
    L.off_gbase = L.off_ghist + (int64_t)kMaxPasses * kRadix * 8;
    L.off_status = L.off_gbase + (int64_t)kMaxPasses * kRadix * 8;
    L.control_bytes = L.off_status + round_up(2 * L.tiles * kRadix * (L.wide_status ? 8 : 4), 256);
    L.off_keys = L.control_bytes;
    L.off_values = L.off_keys + round_up(n * key_bytes, 256);
    L.total = L.off_values + round_up(n * value_bytes, 256);
    return L;
}

// Opts the kernel in to its dynamic shared memory and asks how many of its blocks fit on one
// SM; once per kernel instantiation and CUDA context (function attributes belong to a context).
template <typename KernelT>
static int configure_persistent(KernelT kernel, int threads, size_t bytes, int *blocks_per_sm) {
    static ContextCache<int> cache;
    int blocks = 0;
    if (!cache.find(&blocks)) {
        B200ALG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        // all of the SM's L1 / shared-memory array as shared memory: two blocks need more than
        // the split the driver would pick by itself
        B200ALG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        B200ALG_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, threads, bytes));
        if (blocks < 1) return B200ALG_UNSUPPORTED;
        cache.store(blocks);
    }
    *blocks_per_sm = blocks;
    return B200ALG_OK;
}

// Measurement hook (b200alg_testing_time_sort_pass): events recorded around one digit pass of
// the calling thread's next sort.
thread_local cudaEvent_t g_timed_pass_events[2] = {nullptr, nullptr};
thread_local int g_timed_pass = -1;

// What a sort call works on, untyped (the entry points fill this in).
struct SortCall {
    const void *in_keys;
    void *out_keys;
    const void *in_values;
    void *out_values;
    int64_t stride;
    int64_t n;                  // element count, or its upper bound when n_device is set
    const long long *n_device;
    int value_seq;
    bool out_of_place;
};

template <typename K, typename V, typename SW, typename XF>
static int run_passes(cudaStream_t s, const SortCall &call, const KeyXform<K> &xf, void *temp, const SortLayout &L) {
    constexpr int THREADS = SortTuning<K>::THREADS, ITEMS = SortTuning<K>::ITEMS;
    using Smem = OnesweepSmem<K, V, false, THREADS, ITEMS>;
    auto kernel = onesweep_kernel<K, V, SW, RadixDigit<K, XF>, THREADS, ITEMS>;
    int blocks_per_sm = 0;
    {
        const int rc = configure_persistent(kernel, THREADS, Smem::bytes, &blocks_per_sm);
        if (rc != B200ALG_OK) return rc;
    }
    const int64_t n = call.n;
    const int64_t resident = (int64_t)sm_count() * blocks_per_sm;
    const int grid = (int)(L.tiles < resident ? L.tiles : resident);
    char *t = (char *)temp;
    TempHeader *hdr = (TempHeader *)temp;
    unsigned long long *ghist = (unsigned long long *)(t + L.off_ghist);
    unsigned long long *gbase = (unsigned long long *)(t + L.off_gbase);
    SW *status = (SW *)(t + L.off_status);
    SortBuffers<K, V> io;
    io.in = (const K *)call.in_keys;
    io.out = (K *)call.out_keys;
    io.alt = (K *)(t + L.off_keys);
    io.vin = (const V *)call.in_values;
    io.vout = (V *)call.out_values;
    io.valt = (V *)(t + L.off_values);
    io.stride = call.stride;
    io.n = n;
    io.n_device = call.n_device;

    B200ALG_CUDA_TRY(cudaMemsetAsync(temp, 0, (size_t)L.control_bytes, s));
    {
        const int64_t per_block = (int64_t)kHistoThreads * (16 / sizeof(K)) * 2;
        int64_t want = ceil_div(n, per_block);
        // 32 counter replicas for long inputs (16 for 8-byte keys: 128 KB either way), else 8
        constexpr int kBigShift = sizeof(K) == 8 ? 4 : 5;
        const bool big = n >= (1ll << 22);
        const size_t histo_smem = (size_t)sizeof(K) * kRadix * sizeof(unsigned int) << (big ? kBigShift : 3);
        const int64_t cap = (int64_t)sm_count() * (histo_smem > 100 * 1024 ? 1 : 2);
        const int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
        {
            static ContextCache<int> opted_in;
            int done = 0;
            if (!opted_in.find(&done)) {
                B200ALG_CUDA_TRY(cudaFuncSetAttribute(sort_histogram_kernel<K, kBigShift>, cudaFuncAttributeMaxDynamicSharedMemorySize, kHistoMaxSmem));
                B200ALG_CUDA_TRY(cudaFuncSetAttribute(sort_histogram_kernel<K, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, kHistoMaxSmem));
                opted_in.store(1);
            }
        }
        if (big)
            sort_histogram_kernel<K, kBigShift><<<blocks, kHistoThreads, histo_smem, s>>>(io.in, io.stride, n, io.n_device, xf, ghist);
        else
            sort_histogram_kernel<K, 3><<<blocks, kHistoThreads, histo_smem, s>>>(io.in, io.stride, n, io.n_device, xf, ghist);
        B200ALG_LAUNCH_CHECK();
    }
    sort_offsets_kernel<<<1, kRadix, 0, s>>>(ghist, gbase, hdr, L.passes, (long long)n, io.n_device, 1, call.out_of_place ? 1 : 0);
    B200ALG_LAUNCH_CHECK();
    for (int p = 0; p < L.passes; ++p) {
        RadixDigit<K, XF> dg;
        if constexpr (std::is_same<XF, KeyXform<K>>::value) dg.xf = xf;
        dg.shift = p * 8;
        if (g_timed_pass == p) B200ALG_CUDA_TRY(cudaEventRecord(g_timed_pass_events[0], s));
        if (kSortPdl) {
            B200ALG_CUDA_TRY(launch_dependent(kernel, dim3(grid), dim3(THREADS), Smem::bytes, s, io, p, dg, hdr,
                                              (const unsigned long long *)gbase, status, (int)L.tiles, call.value_seq));
        } else {
            kernel<<<grid, THREADS, Smem::bytes, s>>>(io, p, dg, hdr, gbase, status, (int)L.tiles, call.value_seq);
            B200ALG_LAUNCH_CHECK();
        }
        if (g_timed_pass == p) B200ALG_CUDA_TRY(cudaEventRecord(g_timed_pass_events[1], s));
    }
    {
        int64_t want = ceil_div(n, 256 * 8);
        const int64_t cap = (int64_t)sm_count() * 8;
        const int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
        sort_copy_back_kernel<K, V><<<blocks, 256, 0, s>>>(io, hdr, call.value_seq);
        B200ALG_LAUNCH_CHECK();
    }
    return B200ALG_OK;
}

template <typename K, typename V>
static int run_sort(cudaStream_t s, const SortCall &call, uint64_t xn, uint64_t xp, void *temp, const SortLayout &L) {
    KeyXform<K> xf{(K)xn, (K)xp};
    const bool identity = xn == 0 && xp == 0;
    if (L.wide_status) {
        if (identity) return run_passes<K, V, unsigned long long, KeyIdentity<K>>(s, call, xf, temp, L);
        return run_passes<K, V, unsigned long long, KeyXform<K>>(s, call, xf, temp, L);
    }
    if (identity) return run_passes<K, V, unsigned int, KeyIdentity<K>>(s, call, xf, temp, L);
    return run_passes<K, V, unsigned int, KeyXform<K>>(s, call, xf, temp, L);
}

template <typename V>
static int dispatch_key(cudaStream_t s, int key_bytes, const SortCall &call, uint64_t xn, uint64_t xp, void *temp,
                        const SortLayout &L) {
    switch (key_bytes) {
    case 1: return run_sort<uint8_t, V>(s, call, xn, xp, temp, L);
    case 2: return run_sort<uint16_t, V>(s, call, xn, xp, temp, L);
    case 4: return run_sort<uint32_t, V>(s, call, xn, xp, temp, L);
    case 8: return run_sort<uint64_t, V>(s, call, xn, xp, temp, L);
    }
    return B200ALG_UNSUPPORTED;
}

// ---- 5. stable partition of a shard into per-rank buckets (multi-GPU sort) ---------------
// Bucket sizes of a shard.  With at most eight buckets (one per rank) every thread counts in
// a register, one byte per bucket, and empties it into 32-bit totals before a byte can wrap;
// the totals are added up per warp by shuffles and per block in shared memory.  More buckets
// than that are counted with shared-memory atomics on tables private to each warp.
template <typename K>
__global__ void __launch_bounds__(256)
bucket_histogram_kernel(const K *__restrict__ keys, int64_t n, SplitterBucket<K> dg, unsigned long long *ghist) {
    __shared__ unsigned int sh[8][kRadix];
    __shared__ __align__(16) unsigned char tables[SplitterBucket<K>::kTableBytesWithoutPointers];
    dg.stage(tables, false);
    for (int i = threadIdx.x; i < 8 * kRadix; i += 256) (&sh[0][0])[i] = 0u;
    __syncthreads();
    unsigned int *mine = sh[threadIdx.x >> 5];
    const int64_t step = (int64_t)gridDim.x * 256;
    const int64_t gtid = (int64_t)blockIdx.x * 256 + threadIdx.x;

    auto count_few = [&](auto slots) {
        constexpr int SLOTS = decltype(slots)::value;
        auto bucket = [&](K key, int64_t index) {
            bool tie;
            unsigned int d = dg.template few<SLOTS>(key, tables, tie);
            if (tie) d = SplitterBucket<K>::resolve_tie(dg.xf, dg.index_base, dg.num_splitters, key, index, tables, d);
            return d;
        };
        constexpr int VEC = 16 / (int)sizeof(K);
        union Pack { uint4 u; K k[VEC]; };
        int64_t head = (int64_t)(((16u - (unsigned)((uintptr_t)keys & 15u)) & 15u) / sizeof(K));
        if (head > n) head = n;
        const uint4 *vin = reinterpret_cast<const uint4 *>(keys + head);
        const int64_t nvec = (n - head) / VEC;
        const int64_t tail = head + nvec * VEC;
        unsigned long long bytes = 0ull;  // byte b = keys of bucket b since the last flush
        unsigned int total[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        int pending = 0;
        auto flush = [&]() {
#pragma unroll
            for (int b = 0; b < 8; ++b) total[b] += (unsigned int)(bytes >> (8 * b)) & 0xFFu;
            bytes = 0ull;
            pending = 0;
        };
        int64_t v = gtid;
        for (; v + step < nvec; v += 2 * step) {  // two 16-byte loads in flight per thread (four measured slower)
            Pack a, b;
            a.u = __ldcs(vin + v);
            b.u = __ldcs(vin + v + step);
#pragma unroll
            for (int k = 0; k < VEC; ++k) bytes += 1ull << (8 * bucket(a.k[k], head + v * VEC + k));
#pragma unroll
            for (int k = 0; k < VEC; ++k) bytes += 1ull << (8 * bucket(b.k[k], head + (v + step) * VEC + k));
            pending += 2 * VEC;
            if (pending > 255 - 2 * VEC) flush();
        }
        for (; v < nvec; v += step) {
            Pack a;
            a.u = __ldcs(vin + v);
#pragma unroll
            for (int k = 0; k < VEC; ++k) bytes += 1ull << (8 * bucket(a.k[k], head + v * VEC + k));
            pending += VEC;
            if (pending > 255 - 2 * VEC) flush();
        }
        if (blockIdx.x == 0) {  // the unaligned ends: fewer than 16 bytes each
            if (threadIdx.x < head) bytes += 1ull << (8 * bucket(keys[threadIdx.x], threadIdx.x));
            const int64_t j = tail + threadIdx.x;
            if (j < n) bytes += 1ull << (8 * bucket(keys[j], j));
        }
        flush();
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            unsigned int t = total[b];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) t += __shfl_down_sync(0xffffffffu, t, d);
            if ((threadIdx.x & 31) == 0 && t) mine[b] = t;
        }
    };
    const int ns = dg.num_splitters;  // uniform over the grid
    if (ns <= 1) count_few(std::integral_constant<int, 1>{});
    else if (ns <= 3) count_few(std::integral_constant<int, 3>{});
    else if (ns <= SplitterBucket<K>::kSmall) count_few(std::integral_constant<int, 7>{});
    else {
        for (int64_t i = gtid; i < n; i += step) atomicAdd(mine + dg(keys[i], i, tables), 1u);
    }
    __syncthreads();
    unsigned int c = 0;
#pragma unroll
    for (int r = 0; r < 8; ++r) c += sh[r][threadIdx.x];
    if (c) atomicAdd(ghist + threadIdx.x, (unsigned long long)c);
}

__global__ void export_bucket_counts_kernel(const unsigned long long *ghist, int64_t *counts, int num_buckets) {
    if ((int)threadIdx.x < num_buckets) counts[threadIdx.x] = (int64_t)ghist[threadIdx.x];
}

template <typename K, typename V, typename SW>
static int run_partition(cudaStream_t s, const K *keys, const V *values, int64_t n, const SplitterBucket<K> &dg,
                         K *out_keys, V *out_values, int64_t *counts, int num_buckets, void *temp, const SortLayout &L) {
    constexpr int THREADS = SortTuning<K>::THREADS, ITEMS = SortTuning<K>::ITEMS;
    using Smem = OnesweepSmem<K, V, true, THREADS, ITEMS>;
    auto kernel = onesweep_kernel<K, V, SW, SplitterBucket<K>, THREADS, ITEMS>;
    int blocks_per_sm = 0;
    {
        const int rc = configure_persistent(kernel, THREADS, Smem::bytes, &blocks_per_sm);
        if (rc != B200ALG_OK) return rc;
    }
    const int64_t resident = (int64_t)sm_count() * blocks_per_sm;
    const int grid = (int)(L.tiles < resident ? L.tiles : resident);
    char *t = (char *)temp;
    TempHeader *hdr = (TempHeader *)temp;
    unsigned long long *ghist = (unsigned long long *)(t + L.off_ghist);
    unsigned long long *gbase = (unsigned long long *)(t + L.off_gbase);
    SW *status = (SW *)(t + L.off_status);
    B200ALG_CUDA_TRY(cudaMemsetAsync(temp, 0, (size_t)L.control_bytes, s));
    {
        int64_t want = ceil_div(n, 256 * 8);
        const int64_t cap = (int64_t)sm_count() * 8;
        const int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
        bucket_histogram_kernel<K><<<blocks, 256, 0, s>>>(keys, n, dg, ghist);
        B200ALG_LAUNCH_CHECK();
    }
    // One "pass": offsets of the buckets; the skip rule is off (n + 1 never matches a count),
    // so the pass always moves the keys from buffer 0 (input) to buffer 1 (output).
    sort_offsets_kernel<<<1, kRadix, 0, s>>>(ghist, gbase, hdr, 1, (long long)n, nullptr, 0, 1);
    B200ALG_LAUNCH_CHECK();
    export_bucket_counts_kernel<<<1, kRadix, 0, s>>>(ghist, counts, num_buckets);
    B200ALG_LAUNCH_CHECK();
    SortBuffers<K, V> io{keys, out_keys, nullptr, values, out_values, nullptr, 1, n, nullptr};
    kernel<<<grid, THREADS, Smem::bytes, s>>>(io, 0, dg, hdr, gbase, status, (int)L.tiles, (int)kSeqNone);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

// Bucket sizes only (the first half of a partition whose second half scatters to peers).
template <typename K>
static int run_bucket_count(cudaStream_t s, const K *keys, int64_t n, const SplitterBucket<K> &dg, int64_t *counts,
                            int num_buckets, void *temp, const SortLayout &L) {
    unsigned long long *ghist = (unsigned long long *)((char *)temp + L.off_ghist);
    B200ALG_CUDA_TRY(cudaMemsetAsync(ghist, 0, kRadix * sizeof(unsigned long long), s));
    int64_t want = ceil_div(n, 256 * 8);
    const int64_t cap = (int64_t)sm_count() * 8;
    const int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    bucket_histogram_kernel<K><<<blocks, 256, 0, s>>>(keys, n, dg, ghist);
    B200ALG_LAUNCH_CHECK();
    export_bucket_counts_kernel<<<1, kRadix, 0, s>>>(ghist, counts, num_buckets);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

// The partition pass with one destination per bucket (dg.bucket_keys / dg.bucket_values).
template <typename K, typename V, typename SW>
static int run_bucket_scatter(cudaStream_t s, const K *keys, const V *values, int64_t n, const SplitterBucket<K> &dg,
                              void *temp, const SortLayout &L) {
    constexpr int THREADS = SortTuning<K>::THREADS, ITEMS = SortTuning<K>::ITEMS;
    using Smem = OnesweepSmem<K, V, true, THREADS, ITEMS>;
    auto kernel = onesweep_kernel<K, V, SW, SplitterBucket<K>, THREADS, ITEMS>;
    int blocks_per_sm = 0;
    {
        const int rc = configure_persistent(kernel, THREADS, Smem::bytes, &blocks_per_sm);
        if (rc != B200ALG_OK) return rc;
    }
    const int64_t resident = (int64_t)sm_count() * blocks_per_sm;
    const int grid = (int)(L.tiles < resident ? L.tiles : resident);
    char *t = (char *)temp;
    TempHeader *hdr = (TempHeader *)temp;
    unsigned long long *ghist = (unsigned long long *)(t + L.off_ghist);
    unsigned long long *gbase = (unsigned long long *)(t + L.off_gbase);
    SW *status = (SW *)(t + L.off_status);
    B200ALG_CUDA_TRY(cudaMemsetAsync(temp, 0, (size_t)L.control_bytes, s));
    // all-zero histogram: the bucket offsets come out zero (every bucket has its own base
    // pointer) and the pass is scheduled from buffer 0
    sort_offsets_kernel<<<1, kRadix, 0, s>>>(ghist, gbase, hdr, 1, (long long)n, nullptr, 0, 1);
    B200ALG_LAUNCH_CHECK();
    SortBuffers<K, V> io{keys, nullptr, nullptr, values, nullptr, nullptr, 1, n, nullptr};
    kernel<<<grid, THREADS, Smem::bytes, s>>>(io, 0, dg, hdr, gbase, status, (int)L.tiles, (int)kSeqNone);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

template <typename K, typename V>
static int scatter_typed(cudaStream_t s, const void *keys, const void *values, int64_t n, const SplitterBucket<K> &dg, void *temp,
                         const SortLayout &L) {
    if (L.wide_status) return run_bucket_scatter<K, V, unsigned long long>(s, (const K *)keys, (const V *)values, n, dg, temp, L);
    return run_bucket_scatter<K, V, unsigned int>(s, (const K *)keys, (const V *)values, n, dg, temp, L);
}

template <typename K>
static int bucket_ops_for_key(cudaStream_t s, bool scatter, const void *keys, const void *values, int64_t n, int value_bytes,
                              uint64_t xn, uint64_t xp, const void *sk, const int64_t *si, int ns, int64_t base,
                              void *const *bucket_keys, void *const *bucket_values, int64_t *counts, void *temp,
                              const SortLayout &L) {
    SplitterBucket<K> dg{KeyXform<K>{(K)xn, (K)xp}, (const K *)sk, si, ns, base, bucket_keys, bucket_values};
    if (!scatter) return run_bucket_count<K>(s, (const K *)keys, n, dg, counts, ns + 1, temp, L);
    switch (value_bytes) {
    case 0: return scatter_typed<K, NoValue>(s, keys, values, n, dg, temp, L);
    case 4: return scatter_typed<K, uint32_t>(s, keys, values, n, dg, temp, L);
    case 8: return scatter_typed<K, uint64_t>(s, keys, values, n, dg, temp, L);
    }
    return B200ALG_UNSUPPORTED;
}

static int bucket_ops(void *stream, bool scatter, const void *keys, const void *values, int64_t n, int key_dtype, int value_bytes,
                      int order, const void *splitter_keys, const int64_t *splitter_index, int num_splitters,
                      int64_t index_base, void *const *bucket_keys, void *const *bucket_values, int64_t *counts, void *temp,
                      int64_t temp_bytes) {
    if (!keys || !temp) return B200ALG_INVALID_ARGUMENT;
    if (n < 0 || num_splitters < 0 || num_splitters > 254) return B200ALG_INVALID_ARGUMENT;
    if (num_splitters && (!splitter_keys || !splitter_index)) return B200ALG_INVALID_ARGUMENT;
    const int kb = dtype_bytes(key_dtype);
    if (kb == 0) return B200ALG_UNSUPPORTED;
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
    if (((uintptr_t)keys % kb) || ((uintptr_t)temp % 256)) return B200ALG_MISALIGNED;
    uint64_t xn, xp;
    if (!key_xform_constants(key_dtype, order, xn, xp)) return B200ALG_UNSUPPORTED;
    const SortLayout L = sort_layout(kb, 0, n);
    if (temp_bytes < L.control_bytes) return B200ALG_TEMP_TOO_SMALL;
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) {
        if (!scatter) B200ALG_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int64_t) * (num_splitters + 1), s));
        return B200ALG_OK;
    }
    switch (kb) {
    case 1: return bucket_ops_for_key<uint8_t>(s, scatter, keys, values, n, value_bytes, xn, xp, splitter_keys, splitter_index, num_splitters, index_base, bucket_keys, bucket_values, counts, temp, L);
    case 2: return bucket_ops_for_key<uint16_t>(s, scatter, keys, values, n, value_bytes, xn, xp, splitter_keys, splitter_index, num_splitters, index_base, bucket_keys, bucket_values, counts, temp, L);
    case 4: return bucket_ops_for_key<uint32_t>(s, scatter, keys, values, n, value_bytes, xn, xp, splitter_keys, splitter_index, num_splitters, index_base, bucket_keys, bucket_values, counts, temp, L);
    case 8: return bucket_ops_for_key<uint64_t>(s, scatter, keys, values, n, value_bytes, xn, xp, splitter_keys, splitter_index, num_splitters, index_base, bucket_keys, bucket_values, counts, temp, L);
    }
    return B200ALG_UNSUPPORTED;
}

template <typename K, typename V>
static int partition_typed(cudaStream_t s, const void *keys, const void *values, int64_t n, uint64_t xn, uint64_t xp,
                           const void *splitter_keys, const int64_t *splitter_index, int num_splitters,
                           int64_t index_base, void *out_keys, void *out_values, int64_t *counts, void *temp,
                           const SortLayout &L) {
    SplitterBucket<K> dg{KeyXform<K>{(K)xn, (K)xp}, (const K *)splitter_keys, splitter_index, num_splitters, index_base,
                         nullptr, nullptr};
    if (L.wide_status)
        return run_partition<K, V, unsigned long long>(s, (const K *)keys, (const V *)values, n, dg, (K *)out_keys,
                                                       (V *)out_values, counts, num_splitters + 1, temp, L);
    return run_partition<K, V, unsigned int>(s, (const K *)keys, (const V *)values, n, dg, (K *)out_keys, (V *)out_values,
                                             counts, num_splitters + 1, temp, L);
}

template <typename V>
static int partition_key(cudaStream_t s, int kb, const void *keys, const void *values, int64_t n, uint64_t xn, uint64_t xp,
                         const void *sk, const int64_t *si, int ns, int64_t base, void *ok, void *ov, int64_t *counts,
                         void *temp, const SortLayout &L) {
    switch (kb) {
    case 1: return partition_typed<uint8_t, V>(s, keys, values, n, xn, xp, sk, si, ns, base, ok, ov, counts, temp, L);
    case 2: return partition_typed<uint16_t, V>(s, keys, values, n, xn, xp, sk, si, ns, base, ok, ov, counts, temp, L);
    case 4: return partition_typed<uint32_t, V>(s, keys, values, n, xn, xp, sk, si, ns, base, ok, ov, counts, temp, L);
    case 8: return partition_typed<uint64_t, V>(s, keys, values, n, xn, xp, sk, si, ns, base, ok, ov, counts, temp, L);
    }
    return B200ALG_UNSUPPORTED;
}

static int sort_common(void *stream, const SortCall &call, int key_dtype, int value_bytes, int order, void *temp,
                       int64_t temp_bytes) {
    // Argument checks mirror VerifyArguments (RadixSortExtensions.cs:1340-1367).
    if (!call.in_keys || !call.out_keys || !temp || (value_bytes && !call.out_values)) return B200ALG_INVALID_ARGUMENT;
    if (value_bytes && !call.in_values && call.value_seq == kSeqNone) return B200ALG_INVALID_ARGUMENT;
    if (call.n < 0 || call.stride < 1) return B200ALG_INVALID_ARGUMENT;
    const int kb = dtype_bytes(key_dtype);
    if (kb == 0) return B200ALG_UNSUPPORTED;
    if (value_bytes != 0 && value_bytes != 1 && value_bytes != 2 && value_bytes != 4 && value_bytes != 8 && value_bytes != 16)
        return B200ALG_UNSUPPORTED;
    if (call.value_seq != kSeqNone && value_bytes == 16) return B200ALG_UNSUPPORTED;
    if (call.n > kMaxElements) return B200ALG_TOO_LARGE;
    if (((uintptr_t)call.in_keys % kb) || ((uintptr_t)call.out_keys % kb) || ((uintptr_t)temp % 256)) return B200ALG_MISALIGNED;
    if (value_bytes && (((uintptr_t)call.in_values % value_bytes) || ((uintptr_t)call.out_values % value_bytes)))
        return B200ALG_MISALIGNED;
    if (call.n_device && ((uintptr_t)call.n_device % 8)) return B200ALG_MISALIGNED;
    uint64_t xn, xp;
    if (!key_xform_constants(key_dtype, order, xn, xp)) return B200ALG_UNSUPPORTED;
    const SortLayout L = sort_layout(kb, value_bytes, call.n);
    if (temp_bytes < L.total) return B200ALG_TEMP_TOO_SMALL;
    if (call.n == 0) return B200ALG_OK;
    cudaStream_t s = (cudaStream_t)stream;
    switch (value_bytes) {
    case 0: return dispatch_key<NoValue>(s, kb, call, xn, xp, temp, L);
    case 1: return dispatch_key<uint8_t>(s, kb, call, xn, xp, temp, L);
    case 2: return dispatch_key<uint16_t>(s, kb, call, xn, xp, temp, L);
    case 4: return dispatch_key<uint32_t>(s, kb, call, xn, xp, temp, L);
    case 8: return dispatch_key<uint64_t>(s, kb, call, xn, xp, temp, L);
    case 16: return dispatch_key<uint4>(s, kb, call, xn, xp, temp, L);
    }
    return B200ALG_UNSUPPORTED;
}

}  // namespace b200alg

using namespace b200alg;

extern "C" int b200alg_radix_sort_temp_bytes(int key_dtype, int64_t n, int value_bytes, int64_t *out_bytes) {
    if (!out_bytes || n < 0 || value_bytes < 0) return B200ALG_INVALID_ARGUMENT;
    const int kb = dtype_bytes(key_dtype);
    if (kb == 0) return B200ALG_UNSUPPORTED;
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
    *out_bytes = sort_layout(kb, value_bytes, n).total;
    return B200ALG_OK;
}

extern "C" int b200alg_radix_sort_keys(void *stream, void *keys, int64_t n, int64_t stride, int key_dtype, int order,
                                       void *temp, int64_t temp_bytes) {
    const SortCall call{keys, keys, nullptr, nullptr, stride, n, nullptr, kSeqNone, false};
    return sort_common(stream, call, key_dtype, 0, order, temp, temp_bytes);
}

extern "C" int b200alg_radix_sort_pairs(void *stream, void *keys, void *values, int64_t n, int key_dtype, int value_bytes,
                                        int order, void *temp, int64_t temp_bytes) {
    if (value_bytes == 0) return B200ALG_INVALID_ARGUMENT;
    const SortCall call{keys, keys, values, values, 1, n, nullptr, kSeqNone, false};
    return sort_common(stream, call, key_dtype, value_bytes, order, temp, temp_bytes);
}

extern "C" int b200alg_radix_sort_out_of_place(void *stream, const void *in_keys, const void *in_values, void *out_keys,
                                               void *out_values, int64_t n, const int64_t *n_device, int key_dtype,
                                               int value_bytes, int order, void *temp, int64_t temp_bytes) {
    if (in_keys == out_keys || (value_bytes && in_values == out_values)) return B200ALG_INVALID_ARGUMENT;
    const SortCall call{in_keys, out_keys, in_values, out_values, 1, n, (const long long *)n_device, kSeqNone, true};
    return sort_common(stream, call, key_dtype, value_bytes, order, temp, temp_bytes);
}

extern "C" int b200alg_radix_sort_pairs_sequence(void *stream, void *keys, void *values, int64_t n, int key_dtype,
                                                 int value_dtype, int order, void *temp, int64_t temp_bytes) {
    const int vb = dtype_bytes(value_dtype);
    if (vb == 0) return B200ALG_UNSUPPORTED;
    const bool floating = value_dtype == B200ALG_F16 || value_dtype == B200ALG_F32 || value_dtype == B200ALG_F64;
    const SortCall call{keys, keys, values, values, 1, n, nullptr, floating ? kSeqFloating : kSeqInteger, false};
    return sort_common(stream, call, key_dtype, vb, order, temp, temp_bytes);
}

extern "C" int b200alg_testing_time_sort_pass(void *stream, void *keys, int64_t n, int key_dtype, int order, void *temp,
                                              int64_t temp_bytes, int pass, float *milliseconds) {
    if (!milliseconds || pass < 0 || pass >= kMaxPasses) return B200ALG_INVALID_ARGUMENT;
    cudaEvent_t ev[2];
    B200ALG_CUDA_TRY(cudaEventCreate(&ev[0]));
    B200ALG_CUDA_TRY(cudaEventCreate(&ev[1]));
    g_timed_pass_events[0] = ev[0];
    g_timed_pass_events[1] = ev[1];
    g_timed_pass = pass;
    const int rc = b200alg_radix_sort_keys(stream, keys, n, 1, key_dtype, order, temp, temp_bytes);
    g_timed_pass = -1;
    int result = rc;
    if (rc == B200ALG_OK) {
        if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess || cudaEventElapsedTime(milliseconds, ev[0], ev[1]) != cudaSuccess)
            result = B200ALG_CUDA_ERROR;
    }
    cudaEventDestroy(ev[0]);
    cudaEventDestroy(ev[1]);
    return result;
}

extern "C" int b200alg_bucket_partition_temp_bytes(int key_dtype, int64_t n, int64_t *out_bytes) {
    if (!out_bytes || n < 0) return B200ALG_INVALID_ARGUMENT;
    const int kb = dtype_bytes(key_dtype);
    if (kb == 0) return B200ALG_UNSUPPORTED;
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
    *out_bytes = sort_layout(kb, 0, n).control_bytes;
    return B200ALG_OK;
}

extern "C" int b200alg_bucket_partition(void *stream, const void *keys, const void *values, int64_t n, int key_dtype,
                                        int value_bytes, int order, const void *splitter_keys,
                                        const int64_t *splitter_index, int num_splitters, int64_t index_base,
                                        void *out_keys, void *out_values, int64_t *bucket_counts, void *temp,
                                        int64_t temp_bytes) {
    if (!keys || !out_keys || !bucket_counts || !temp) return B200ALG_INVALID_ARGUMENT;
    if (value_bytes && (!values || !out_values)) return B200ALG_INVALID_ARGUMENT;
    if (n < 0 || num_splitters < 0 || num_splitters > 254) return B200ALG_INVALID_ARGUMENT;
    if (num_splitters && (!splitter_keys || !splitter_index)) return B200ALG_INVALID_ARGUMENT;
    const int kb = dtype_bytes(key_dtype);
    if (kb == 0) return B200ALG_UNSUPPORTED;
    if (value_bytes != 0 && value_bytes != 4 && value_bytes != 8) return B200ALG_UNSUPPORTED;
    if (n > kMaxElements) return B200ALG_TOO_LARGE;
    if (((uintptr_t)keys % kb) || ((uintptr_t)out_keys % kb) || ((uintptr_t)temp % 256) || ((uintptr_t)bucket_counts % 8))
        return B200ALG_MISALIGNED;
    uint64_t xn, xp;
    if (!key_xform_constants(key_dtype, order, xn, xp)) return B200ALG_UNSUPPORTED;
    const SortLayout L = sort_layout(kb, 0, n);
    if (temp_bytes < L.control_bytes) return B200ALG_TEMP_TOO_SMALL;
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) {
        B200ALG_CUDA_TRY(cudaMemsetAsync(bucket_counts, 0, sizeof(int64_t) * (num_splitters + 1), s));
        return B200ALG_OK;
    }
    switch (value_bytes) {
    case 0: return partition_key<NoValue>(s, kb, keys, values, n, xn, xp, splitter_keys, splitter_index, num_splitters,
                                          index_base, out_keys, out_values, bucket_counts, temp, L);
    case 4: return partition_key<uint32_t>(s, kb, keys, values, n, xn, xp, splitter_keys, splitter_index, num_splitters,
                                           index_base, out_keys, out_values, bucket_counts, temp, L);
    case 8: return partition_key<uint64_t>(s, kb, keys, values, n, xn, xp, splitter_keys, splitter_index, num_splitters,
                                           index_base, out_keys, out_values, bucket_counts, temp, L);
    }
    return B200ALG_UNSUPPORTED;
}

// ---- 6. splitters out of a sample, without sorting it --------------------------------------
// Pair t's rank is the number of pairs in front of it in the order (transformed key, slot):
// what a stable sort by key would give.  A block holds 256 pairs and counts against a slab of
// kSelectSlab pairs in shared memory; the partial ranks meet in global memory.
constexpr int kSelectSlab = 1024;
constexpr int64_t kSelectMax = 1 << 16;

template <typename K>
__global__ void __launch_bounds__(256)
sample_rank_kernel(const K *__restrict__ keys, const long long *m_device, int64_t max_m, KeyXform<K> xf, unsigned int *ranks) {
    __shared__ K slab[kSelectSlab];
    long long m = *m_device;
    m = m < 0 ? 0 : (m > max_m ? max_m : m);
    const int64_t first = (int64_t)blockIdx.x * 256, slab_first = (int64_t)blockIdx.y * kSelectSlab;
    if (first >= m || slab_first >= m) return;
    const int len = (int)(m - slab_first < kSelectSlab ? m - slab_first : kSelectSlab);
    for (int j = threadIdx.x; j < len; j += 256) slab[j] = xf(keys[slab_first + j]);
    __syncthreads();
    const int64_t t = first + threadIdx.x;
    if (t >= m) return;
    const K mine = xf(keys[t]);
    // slots of the slab in front of t break ties in their favour, the others do not
    const int split = (int)(t - slab_first < 0 ? 0 : (t - slab_first > len ? len : t - slab_first));
    unsigned int r = 0;
    for (int j = 0; j < split; ++j) r += slab[j] <= mine;
    for (int j = split; j < len; ++j) r += slab[j] < mine;
    if (r) atomicAdd(&ranks[t], r);
}

template <typename K>
__global__ void __launch_bounds__(256)
sample_pick_kernel(const K *__restrict__ keys, const int64_t *__restrict__ index, const long long *m_device, int64_t max_m,
                   const unsigned int *ranks, int num_picks, K *out_keys, int64_t *out_index) {
    long long m = *m_device;
    m = m < 0 ? 0 : (m > max_m ? max_m : m);
    const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (m == 0) {
        if (t < num_picks) {
            out_keys[t] = (K)0;
            out_index[t] = 0;
        }
        return;
    }
    if (t >= m) return;
    const long long r = ranks[t];
    for (int j = 0; j < num_picks; ++j) {
        if (((long long)(j + 1) * m) / (num_picks + 1) == r) {
            out_keys[j] = keys[t];
            out_index[j] = index[t];
        }
    }
}

template <typename K>
static int select_typed(cudaStream_t s, const void *keys, const int64_t *index, int64_t max_m, const long long *m_device,
                        uint64_t xn, uint64_t xp, int num_picks, void *out_keys, int64_t *out_index, void *temp) {
    B200ALG_CUDA_TRY(cudaMemsetAsync(temp, 0, (size_t)max_m * 4, s));
    const dim3 grid((unsigned)ceil_div(max_m, 256), (unsigned)ceil_div(max_m, kSelectSlab));
    sample_rank_kernel<K><<<grid, 256, 0, s>>>((const K *)keys, m_device, max_m, KeyXform<K>{(K)xn, (K)xp}, (unsigned int *)temp);
    B200ALG_LAUNCH_CHECK();
    const int64_t threads = max_m > num_picks ? max_m : num_picks;
    sample_pick_kernel<K><<<(unsigned)ceil_div(threads, 256), 256, 0, s>>>((const K *)keys, index, m_device, max_m,
                                                                          (const unsigned int *)temp, num_picks, (K *)out_keys,
                                                                          out_index);
    B200ALG_LAUNCH_CHECK();
    return B200ALG_OK;
}

extern "C" int b200alg_select_splitters(void *stream, const void *keys, const int64_t *index, int64_t max_m,
                                        const int64_t *m_device, int key_dtype, int order, int num_picks, void *out_keys,
                                        int64_t *out_index, void *temp, int64_t temp_bytes) {
    if (!keys || !index || !m_device || !temp || max_m < 1 || num_picks < 0 || num_picks > 254) return B200ALG_INVALID_ARGUMENT;
    if (num_picks && (!out_keys || !out_index)) return B200ALG_INVALID_ARGUMENT;
    if (max_m > kSelectMax) return B200ALG_TOO_LARGE;
    const int kb = dtype_bytes(key_dtype);
    if (kb == 0) return B200ALG_UNSUPPORTED;
    if (((uintptr_t)keys % kb) || ((uintptr_t)out_keys % kb) || ((uintptr_t)temp % 4) || ((uintptr_t)index % 8) ||
        ((uintptr_t)out_index % 8) || ((uintptr_t)m_device % 8))
        return B200ALG_MISALIGNED;
    if (temp_bytes < max_m * 4) return B200ALG_TEMP_TOO_SMALL;
    uint64_t xn, xp;
    if (!key_xform_constants(key_dtype, order, xn, xp)) return B200ALG_UNSUPPORTED;
    if (num_picks == 0) return B200ALG_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long long *m = (const long long *)m_device;
    switch (kb) {
    case 1: return select_typed<uint8_t>(s, keys, index, max_m, m, xn, xp, num_picks, out_keys, out_index, temp);
    case 2: return select_typed<uint16_t>(s, keys, index, max_m, m, xn, xp, num_picks, out_keys, out_index, temp);
    case 4: return select_typed<uint32_t>(s, keys, index, max_m, m, xn, xp, num_picks, out_keys, out_index, temp);
    case 8: return select_typed<uint64_t>(s, keys, index, max_m, m, xn, xp, num_picks, out_keys, out_index, temp);
    }
    return B200ALG_UNSUPPORTED;
}

extern "C" int b200alg_bucket_count(void *stream, const void *keys, int64_t n, int key_dtype, int order,
                                    const void *splitter_keys, const int64_t *splitter_index, int num_splitters,
                                    int64_t index_base, int64_t *bucket_counts, void *temp, int64_t temp_bytes) {
    if (!bucket_counts || ((uintptr_t)bucket_counts % 8)) return B200ALG_INVALID_ARGUMENT;
    return bucket_ops(stream, false, keys, nullptr, n, key_dtype, 0, order, splitter_keys, splitter_index, num_splitters,
                      index_base, nullptr, nullptr, bucket_counts, temp, temp_bytes);
}

extern "C" int b200alg_bucket_scatter(void *stream, const void *keys, const void *values, int64_t n, int key_dtype,
                                      int value_bytes, int order, const void *splitter_keys, const int64_t *splitter_index,
                                      int num_splitters, int64_t index_base, void *const *bucket_key_ptrs,
                                      void *const *bucket_value_ptrs, void *temp, int64_t temp_bytes) {
    if (!bucket_key_ptrs || (value_bytes && (!values || !bucket_value_ptrs))) return B200ALG_INVALID_ARGUMENT;
    if (value_bytes != 0 && value_bytes != 4 && value_bytes != 8) return B200ALG_UNSUPPORTED;
    return bucket_ops(stream, true, keys, values, n, key_dtype, value_bytes, order, splitter_keys, splitter_index,
                      num_splitters, index_base, bucket_key_ptrs, value_bytes ? bucket_value_ptrs : nullptr, nullptr, temp,
                      temp_bytes);
}
