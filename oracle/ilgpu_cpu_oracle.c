/*
 * CPU oracle: a plain-C restatement of the ILGPU.Algorithms CPU-accelerator path for
 * radix sort (keys / pairs), scan, reduce and histogram.
 *
 * THIS IS TEST INFRASTRUCTURE.  It is the checker the CUDA kernels are compared with
 * and the CPU baseline a benchmark may time.  Nothing that ships in the product path
 * may call into this file.
 *
 * Parity pin: the reference's own unit tests hold known-answer cases for this path
 * (ramps of sizes 1/31/33/127/1027, constant arrays, modulo-bin histograms of 1..1024,
 * the overflow scenario); tests/test_oracle_golden.py checks every function below
 * against those cases.  Float *key* ordering is not exercised by the reference's tests
 * with negative or Half values, so for those keys the transform below is a literal
 * reading of the source and counts as "parity unpinned".
 *
 * Each function cites the reference file:line (paths relative to the ILGPU source
 * tree) that it restates.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#include <float.h>
#include <limits.h>

/* dtype / op codes shared with include/b200alg.h */
enum { DT_I8, DT_U8, DT_I16, DT_U16, DT_I32, DT_U32, DT_I64, DT_U64, DT_F16, DT_F32, DT_F64 };
enum { OP_ADD, OP_MAX, OP_MIN };
enum { LOC_EQUAL_WIDTH_CLAMP, LOC_MODULO };

static int dtype_size(int dt) {
    switch (dt) {
    case DT_I8: case DT_U8: return 1;
    case DT_I16: case DT_U16: case DT_F16: return 2;
    case DT_I32: case DT_U32: case DT_F32: return 4;
    case DT_I64: case DT_U64: case DT_F64: return 8;
    }
    return 0;
}

int oracle_dtype_size(int dt) { return dtype_size(dt); }

static uint64_t load_raw(int dt, const void *base, int64_t i) {
    switch (dtype_size(dt)) {
    case 1: return ((const uint8_t *)base)[i];
    case 2: return ((const uint16_t *)base)[i];
    case 4: return ((const uint32_t *)base)[i];
    default: return ((const uint64_t *)base)[i];
    }
}

/* ------------------------------------------------------------------------------------
 * Radix-sort key transform.
 * RadixSortOperations.tt:77-93 (ascending), :122-123 (descending).
 * Returns the value C# calls `bits`, before the shift, as an unsigned 64-bit pattern;
 * only bit positions below NumBits are ever selected by (shift, mask).
 *
 *  - unsigned ints: identity.
 *  - signed ints:   value ^ (1 << (NumBits-1)).
 *  - float/double:  u = FloatAsInt(value) is UNSIGNED (Interop.cs:171-191), so
 *                   (~u >> (NumBits-1)) is a logical shift and yields 0 or 1;
 *                   bits = u ^ (signMask | that).
 *  - Half:          (uint)~u16 >> 15 works on the int-promoted complement, giving
 *                   0x1FFFE | (sign clear ? 1 : 0); bits = u ^ (0x8000 | that).
 * ---------------------------------------------------------------------------------- */
uint64_t oracle_key_bits(int dt, uint64_t raw) {
    switch (dt) {
    case DT_U8: case DT_U16: case DT_U32: case DT_U64:
        return raw;
    case DT_I8:  return (raw ^ 0x80ull) & 0xFFull;
    case DT_I16: return (raw ^ 0x8000ull) & 0xFFFFull;
    case DT_I32: return (raw ^ 0x80000000ull) & 0xFFFFFFFFull;
    case DT_I64: return raw ^ 0x8000000000000000ull;
    case DT_F16: {
        uint32_t u = (uint32_t)(raw & 0xFFFFu);
        uint32_t ones = ((uint32_t)~u) >> 15;           /* 0x1FFFE | !sign */
        uint32_t bits = u ^ (0x8000u | ones);
        return bits & 0xFFFFu;
    }
    case DT_F32: {
        uint32_t u = (uint32_t)raw;
        uint32_t ones = (~u) >> 31;
        return (uint32_t)(u ^ (0x80000000u | ones));
    }
    case DT_F64: {
        uint64_t u = raw;
        uint64_t ones = (~u) >> 63;
        return u ^ (0x8000000000000000ull | ones);
    }
    }
    return raw;
}

/* IRadixSortOperation.ExtractRadixBits (RadixSortOperations.tt:51,92,119-124). */
int oracle_extract_radix_bits(int dt, uint64_t raw, int shift, int mask, int descending) {
    int asc = (int)((oracle_key_bits(dt, raw) >> shift) & (uint64_t)mask);
    return descending ? ((~asc) & mask) : asc;
}

/* ------------------------------------------------------------------------------------
 * Literal radix sort: CPURadixSortKernel1 (RadixSortExtensions.cs:755-826),
 * GetExclusiveCount (:835-836), CPURadixSortKernel2 (:929-979), host loop (:1168-1227):
 * gridDim = accelerator.MaxNumThreads groups of one thread, 2 bits per pass
 * (Specialization4 :988-995), counter[numGroups * bucket + group], inclusive int scan of
 * the counters between the two kernels.  `values` (optional) rides along the way the
 * AoS RadixSortPair does (:477-506, gather/scatter :605-645).
 * ---------------------------------------------------------------------------------- */
int oracle_radix_sort_literal(int dt, void *keys, void *values, int value_bytes, int64_t n,
                              int descending, int num_groups) {
    if (n <= 0) return 0;
    const int U = 4, bit_inc = 2;
    const int ks = dtype_size(dt);
    int64_t iters = (n + num_groups - 1) / num_groups;       /* numIterationsPerGroup */
    uint8_t *tmpk = (uint8_t *)malloc((size_t)n * ks);
    uint8_t *tmpv = values ? (uint8_t *)malloc((size_t)n * value_bytes) : NULL;
    int64_t *counter = (int64_t *)calloc((size_t)num_groups * U, sizeof(int64_t));
    int64_t *counter2 = (int64_t *)calloc((size_t)num_groups * U, sizeof(int64_t));
    uint8_t *k = (uint8_t *)keys, *v = (uint8_t *)values;
    for (int shift = 0; shift < ks * 8; shift += bit_inc) {
        memset(counter, 0, sizeof(int64_t) * num_groups * U);
        /* kernel 1: TileInfo with Group.DimX == 1 (TileInfo.cs:29-35) */
        for (int g = 0; g < num_groups; ++g) {
            int64_t start = (int64_t)g * iters, end = start + iters;
            int64_t maxlen = end < n ? end : n;
            int64_t scan_mem[4] = {0, 0, 0, 0}, add_mem[4] = {0, 0, 0, 0};
            for (int64_t i = start; i < maxlen; ++i)
                ++scan_mem[oracle_extract_radix_bits(dt, load_raw(dt, k, i), shift, U - 1, descending)];
            for (int j = 0; j < U; ++j) counter[(int64_t)num_groups * j + g] = scan_mem[j];
            int64_t scanned = 0, previous = scan_mem[0];
            for (int j = 1; j < U; ++j) { scanned += previous; previous = scan_mem[j]; scan_mem[j] = scanned; }
            scan_mem[0] = 0;
            for (int64_t i = start; i < maxlen; ++i) {
                int b = oracle_extract_radix_bits(dt, load_raw(dt, k, i), shift, U - 1, descending);
                int64_t pos = start + add_mem[b]++ + scan_mem[b];
                memcpy(tmpk + pos * ks, k + i * ks, ks);
                if (v) memcpy(tmpv + pos * value_bytes, v + i * value_bytes, value_bytes);
            }
        }
        /* inclusive AddInt32 scan of the counters (:1204-1208) */
        int64_t run = 0;
        for (int64_t i = 0; i < (int64_t)num_groups * U; ++i) { run += counter[i]; counter2[i] = run; }
        /* kernel 2 */
        for (int g = 0; g < num_groups; ++g) {
            int64_t start = (int64_t)g * iters, end = start + iters;
            int64_t maxlen = end < n ? end : n;
            for (int64_t i = start; i < maxlen; ++i) {
                int b = oracle_extract_radix_bits(dt, load_raw(dt, tmpk, i), shift, U - 1, descending);
                int64_t idx = (int64_t)b * num_groups + g;
                int64_t pos = (idx < 1 ? 0 : counter2[idx - 1]) + i - start;
                int64_t offset = 0;
                for (int w = 0; w < b; ++w) {
                    int64_t a = (int64_t)w * num_groups + g;
                    offset += counter2[a] - (a < 1 ? 0 : counter2[a - 1]);
                }
                pos -= offset;
                memcpy(k + pos * ks, tmpk + i * ks, ks);
                if (v) memcpy(v + pos * value_bytes, tmpv + i * value_bytes, value_bytes);
            }
        }
    }
    free(tmpk); free(tmpv); free(counter); free(counter2);
    return 0;
}

/* ------------------------------------------------------------------------------------
 * Closed form of the sort above for large n: every 2-bit pass is a stable partition by
 * the transformed digit, so the whole sort equals a stable LSD sort by the transformed
 * key (descending: by its complement).  Here with 8-bit digits; test_oracle_golden.py
 * checks it against oracle_radix_sort_literal on random inputs of every key type.
 * ---------------------------------------------------------------------------------- */
int oracle_radix_sort(int dt, void *keys, void *values, int value_bytes, int64_t n, int descending) {
    if (n <= 0) return 0;
    const int ks = dtype_size(dt);
    uint8_t *tmpk = (uint8_t *)malloc((size_t)n * ks);
    uint8_t *tmpv = values ? (uint8_t *)malloc((size_t)n * value_bytes) : NULL;
    uint8_t *srck = (uint8_t *)keys, *dstk = tmpk;
    uint8_t *srcv = (uint8_t *)values, *dstv = tmpv;
    uint64_t flip = descending ? ~0ull : 0ull;
    for (int pass = 0; pass < ks; ++pass) {
        int shift = pass * 8;
        int64_t hist[256];
        memset(hist, 0, sizeof hist);
        for (int64_t i = 0; i < n; ++i)
            ++hist[((oracle_key_bits(dt, load_raw(dt, srck, i)) ^ flip) >> shift) & 0xFF];
        int64_t sum = 0;
        for (int d = 0; d < 256; ++d) { int64_t c = hist[d]; hist[d] = sum; sum += c; }
        switch (ks) {
#define SCATTER(KT)                                                                          \
            for (int64_t i = 0; i < n; ++i) {                                                \
                KT raw = ((const KT *)srck)[i];                                              \
                int64_t pos = hist[((oracle_key_bits(dt, (uint64_t)raw) ^ flip) >> shift) & 0xFF]++; \
                ((KT *)dstk)[pos] = raw;                                                     \
                if (srcv) memcpy(dstv + pos * value_bytes, srcv + i * value_bytes, value_bytes); \
            }
        case 1: SCATTER(uint8_t) break;
        case 2: SCATTER(uint16_t) break;
        case 4: SCATTER(uint32_t) break;
        default: SCATTER(uint64_t) break;
#undef SCATTER
        }
        uint8_t *t = srck; srck = dstk; dstk = t;
        t = srcv; srcv = dstv; dstv = t;
    }
    if (srck != (uint8_t *)keys) {
        memcpy(keys, srck, (size_t)n * ks);
        if (values) memcpy(values, srcv, (size_t)n * value_bytes);
    }
    free(tmpk); free(tmpv);
    return 0;
}

/* ------------------------------------------------------------------------------------
 * Scan / reduce operations: ScanReduceOperations.tt:20-74.
 * Identity: Add 0, Max T.MinValue, Min T.MaxValue.  Apply: first + second (wrapping for
 * ints), XMath.Max / XMath.Min.
 * ---------------------------------------------------------------------------------- */
#define DEFINE_OPS(SFX, T, TMINV, TMAXV)                                                  \
    static T identity_##SFX(int op) { return op == OP_ADD ? (T)0 : (op == OP_MAX ? (TMINV) : (TMAXV)); } \
    static T apply_##SFX(int op, T a, T b) {                                              \
        if (op == OP_ADD) return (T)(a + b);                                              \
        if (op == OP_MAX) return a > b ? a : b;                                           \
        return a < b ? a : b;                                                             \
    }
/* unsigned add keeps C# unchecked wrap-around; signed add is done in unsigned space */
static int32_t identity_i32(int op) { return op == OP_ADD ? 0 : (op == OP_MAX ? INT32_MIN : INT32_MAX); }
static int32_t apply_i32(int op, int32_t a, int32_t b) {
    if (op == OP_ADD) return (int32_t)((uint32_t)a + (uint32_t)b);
    if (op == OP_MAX) return a > b ? a : b;
    return a < b ? a : b;
}
static int64_t identity_i64(int op) { return op == OP_ADD ? 0 : (op == OP_MAX ? INT64_MIN : INT64_MAX); }
static int64_t apply_i64(int op, int64_t a, int64_t b) {
    if (op == OP_ADD) return (int64_t)((uint64_t)a + (uint64_t)b);
    if (op == OP_MAX) return a > b ? a : b;
    return a < b ? a : b;
}
DEFINE_OPS(u32, uint32_t, 0u, UINT32_MAX)
DEFINE_OPS(u64, uint64_t, 0ull, UINT64_MAX)
/* float.MinValue is -FLT_MAX (not -inf) in C#; same for double */
DEFINE_OPS(f32, float, -FLT_MAX, FLT_MAX)
DEFINE_OPS(f64, double, -DBL_MAX, DBL_MAX)

/* ------------------------------------------------------------------------------------
 * Scan: SingleGroupScanKernel (ScanExtensions.cs:407-439) = ComputeTileScan (:340-388)
 * over one tile covering the whole input, with the IL group scan: the first thread scans
 * the group's values serially in shared memory (IL/ILGroupExtensions.cs:116-145);
 * boundaries (:76-106); the carry between chunks is InclusiveScanNextIteration
 * (:184-192) = Apply(left, right) or ExclusiveScanNextIteration (:158-170) =
 * Apply(Apply(left, right), last lane's input).  group_size = MaxNumThreadsPerGroup of
 * the CPU device (16 for the default device, Runtime/CPU/CPUDevice.cs:67-77).
 * Strides are in elements (Stride1D.General).
 * ---------------------------------------------------------------------------------- */
#define DEFINE_SCAN(SFX, T)                                                               \
    static void scan_##SFX(int op, int inclusive, const T *in, int64_t in_stride, T *out, \
                           int64_t out_stride, int64_t n, int group_size) {               \
        T *shared = (T *)malloc(sizeof(T) * (size_t)group_size);                          \
        T *inputs = (T *)malloc(sizeof(T) * (size_t)group_size);                          \
        int64_t iters = (n + group_size - 1) / group_size;                                \
        int64_t end_index = iters * group_size;                                           \
        T left = identity_##SFX(op);                                                      \
        T right = identity_##SFX(op);                                                     \
        for (int64_t base = 0; base < end_index; base += group_size) {                    \
            if (base > 0) {                                                               \
                T next = apply_##SFX(op, left, right);                                    \
                left = inclusive ? next : apply_##SFX(op, next, inputs[group_size - 1]);  \
            }                                                                             \
            for (int t = 0; t < group_size; ++t)                                          \
                inputs[t] = (base + t < n) ? in[(base + t) * in_stride] : identity_##SFX(op); \
            shared[0] = inputs[0];                                                        \
            for (int t = 1; t < group_size; ++t)                                          \
                shared[t] = apply_##SFX(op, shared[t - 1], inputs[t]);                    \
            right = inclusive ? shared[group_size - 1]                                    \
                              : shared[group_size - 2 > 0 ? group_size - 2 : 0];          \
            for (int t = 0; t < group_size; ++t) {                                        \
                if (base + t >= n) continue;                                              \
                T cur = inclusive ? shared[t] : (t == 0 ? identity_##SFX(op) : shared[t - 1]); \
                out[(base + t) * out_stride] = apply_##SFX(op, left, cur);                \
            }                                                                             \
        }                                                                                 \
        free(shared); free(inputs);                                                       \
    }
DEFINE_SCAN(i32, int32_t) DEFINE_SCAN(i64, int64_t) DEFINE_SCAN(u32, uint32_t)
DEFINE_SCAN(u64, uint64_t) DEFINE_SCAN(f32, float) DEFINE_SCAN(f64, double)

int oracle_scan(int dt, int op, int inclusive, const void *in, int64_t in_stride, void *out,
                int64_t out_stride, int64_t n, int group_size) {
    if (n <= 0) return 0;
    if (group_size < 1) return -1;
    switch (dt) {
    case DT_I32: scan_i32(op, inclusive, in, in_stride, out, out_stride, n, group_size); return 0;
    case DT_I64: scan_i64(op, inclusive, in, in_stride, out, out_stride, n, group_size); return 0;
    case DT_U32: scan_u32(op, inclusive, in, in_stride, out, out_stride, n, group_size); return 0;
    case DT_U64: scan_u64(op, inclusive, in, in_stride, out, out_stride, n, group_size); return 0;
    case DT_F32: scan_f32(op, inclusive, in, in_stride, out, out_stride, n, group_size); return 0;
    case DT_F64: scan_f64(op, inclusive, in, in_stride, out, out_stride, n, group_size); return 0;
    }
    return -1;
}

/* ------------------------------------------------------------------------------------
 * Reduce: CreateReduction (ReductionExtensions.cs:135-167) sets output[0] = Identity,
 * then GridStrideLoopKernel (GridExtensions.cs:204-227) runs ReductionImplementation
 * (:52-125): thread t of group g folds elements g*groupDim+t, +gridDim*groupDim, ...;
 * Finish() = group reduce (IL/ILGroupExtensions.cs:35-53: per-warp ShuffleDown tree,
 * PTX/PTXWarpExtensions.cs:26-37, then first lanes AtomicApply into one shared cell that
 * starts at Identity) and one AtomicApply per group into output[0].  Atomic order is
 * unspecified in the reference; this restatement applies warps and groups in index
 * order.  Default CPU device: grid 1, group 16, warp 4.
 * ---------------------------------------------------------------------------------- */
#define DEFINE_REDUCE(SFX, T)                                                             \
    static T reduce_##SFX(int op, const T *in, int64_t stride, int64_t n, int grid_dim,   \
                          int group_dim, int warp_size) {                                 \
        T out = identity_##SFX(op);                                                       \
        T *lane = (T *)malloc(sizeof(T) * (size_t)group_dim);                             \
        int64_t step = (int64_t)grid_dim * group_dim;                                     \
        for (int g = 0; g < grid_dim; ++g) {                                              \
            for (int t = 0; t < group_dim; ++t) {                                         \
                T acc = identity_##SFX(op);                                               \
                for (int64_t i = (int64_t)g * group_dim + t; i < n; i += step)            \
                    acc = apply_##SFX(op, acc, in[i * stride]);                           \
                lane[t] = acc;                                                            \
            }                                                                             \
            T shared = identity_##SFX(op);                                                \
            for (int w = 0; w < group_dim; w += warp_size) {                              \
                for (int off = warp_size / 2; off > 0; off >>= 1)                         \
                    for (int l = 0; l + off < warp_size; ++l)                             \
                        lane[w + l] = apply_##SFX(op, lane[w + l], lane[w + l + off]);    \
                shared = apply_##SFX(op, shared, lane[w]);                                \
            }                                                                             \
            out = apply_##SFX(op, out, shared);                                           \
        }                                                                                 \
        free(lane);                                                                       \
        return out;                                                                       \
    }
DEFINE_REDUCE(i32, int32_t) DEFINE_REDUCE(i64, int64_t) DEFINE_REDUCE(u32, uint32_t)
DEFINE_REDUCE(u64, uint64_t) DEFINE_REDUCE(f32, float) DEFINE_REDUCE(f64, double)

int oracle_reduce(int dt, int op, const void *in, int64_t stride, int64_t n, void *out,
                  int grid_dim, int group_dim, int warp_size) {
    if (n < 1 || grid_dim < 1 || group_dim < 1 || warp_size < 1 || group_dim % warp_size) return -1;
    switch (dt) {
    case DT_I32: *(int32_t *)out = reduce_i32(op, in, stride, n, grid_dim, group_dim, warp_size); return 0;
    case DT_I64: *(int64_t *)out = reduce_i64(op, in, stride, n, grid_dim, group_dim, warp_size); return 0;
    case DT_U32: *(uint32_t *)out = reduce_u32(op, in, stride, n, grid_dim, group_dim, warp_size); return 0;
    case DT_U64: *(uint64_t *)out = reduce_u64(op, in, stride, n, grid_dim, group_dim, warp_size); return 0;
    case DT_F32: *(float *)out = reduce_f32(op, in, stride, n, grid_dim, group_dim, warp_size); return 0;
    case DT_F64: *(double *)out = reduce_f64(op, in, stride, n, grid_dim, group_dim, warp_size); return 0;
    }
    return -1;
}

/* ------------------------------------------------------------------------------------
 * Histogram: HistogramWorkKernel (HistogramExtensions.cs:237-277) through the single-bin
 * adapter (HistogramLaunchers.tt:89-100): bin = locator(value, numBins); old =
 * Atomic.Add(ref histogram[bin], 1); overflow |= (old == T.MaxValue)
 * (HistogramOperations.tt:36-40); the flag is OR-ed into histogramOverflow[0]
 * (HistogramExtensions.cs:197).  The histogram is accumulated into, never cleared.
 *
 * Locators (the reference leaves these to the user; both are named here so that the
 * same arithmetic can run on either side of a C ABI):
 *  - LOC_MODULO: the reference tests' ModuloBin*Operation (HistogramTests.tt:83-94):
 *    ints |value % numBins| (C# truncating remainder), floats |fmod(value, numBins)|
 *    truncated to int.
 *  - LOC_EQUAL_WIDTH_CLAMP: t = (x - lo) * (numBins / (hi - lo)), scale computed once in
 *    the input's float type; b = (int)floor(t) clamped to [0, numBins-1]; NaN -> bin 0.
 *    Integer inputs are converted to double first.
 * ---------------------------------------------------------------------------------- */
static int64_t clamp_bin(double t, int64_t num_bins) {
    if (!(t == t)) return 0;                 /* NaN */
    double f = floor(t);
    if (f < 0.0) return 0;
    if (f >= (double)num_bins) return num_bins - 1;
    return (int64_t)f;
}

int64_t oracle_locate_bin(int dt, uint64_t raw, int locator, double lo, double hi, int64_t num_bins) {
    if (locator == LOC_MODULO) {
        switch (dt) {
        case DT_I32: { int64_t r = (int64_t)(int32_t)raw % num_bins; return r < 0 ? -r : r; }
        case DT_I64: { int64_t r = (int64_t)raw % num_bins; return r < 0 ? -r : r; }
        case DT_U32: return (int64_t)((uint32_t)raw % (uint64_t)num_bins);
        case DT_U64: return (int64_t)(raw % (uint64_t)num_bins);
        case DT_F32: { float f; uint32_t u = (uint32_t)raw; memcpy(&f, &u, 4);
                       return (int64_t)(int32_t)fabsf(fmodf(f, (float)num_bins)); }
        case DT_F64: { double d; memcpy(&d, &raw, 8);
                       return (int64_t)(int32_t)fabs(fmod(d, (double)num_bins)); }
        }
        return -1;
    }
    if (dt == DT_F32) {
        float f; uint32_t u = (uint32_t)raw; memcpy(&f, &u, 4);
        float scale = (float)num_bins / ((float)hi - (float)lo);
        float t = (f - (float)lo) * scale;
        if (!(t == t)) return 0;
        float fl = floorf(t);
        if (fl < 0.0f) return 0;
        if (fl >= (float)num_bins) return num_bins - 1;
        return (int64_t)fl;
    }
    double x;
    switch (dt) {
    case DT_I32: x = (double)(int32_t)raw; break;
    case DT_I64: x = (double)(int64_t)raw; break;
    case DT_U32: x = (double)(uint32_t)raw; break;
    case DT_U64: x = (double)raw; break;
    case DT_F64: memcpy(&x, &raw, 8); break;
    default: return -1;
    }
    double scale = (double)num_bins / (hi - lo);
    return clamp_bin((x - lo) * scale, num_bins);
}

int oracle_histogram(int in_dt, const void *in, int64_t stride, int64_t n, int locator, double lo,
                     double hi, int bin_dt, void *bins, int64_t num_bins, int32_t *overflow) {
    int did_overflow = 0;
    if (num_bins < 1) return -1;
    for (int64_t i = 0; i < n; ++i) {
        int64_t b = oracle_locate_bin(in_dt, load_raw(in_dt, in, i * stride), locator, lo, hi, num_bins);
        if (b < 0 || b >= num_bins) return -2;
        switch (bin_dt) {
        case DT_I32: { int32_t *p = (int32_t *)bins + b; did_overflow |= (*p == INT32_MAX);
                       *p = (int32_t)((uint32_t)*p + 1u); break; }
        case DT_I64: { int64_t *p = (int64_t *)bins + b; did_overflow |= (*p == INT64_MAX);
                       *p = (int64_t)((uint64_t)*p + 1ull); break; }
        case DT_U32: { uint32_t *p = (uint32_t *)bins + b; did_overflow |= (*p == UINT32_MAX); *p += 1u; break; }
        case DT_U64: { uint64_t *p = (uint64_t *)bins + b; did_overflow |= (*p == UINT64_MAX); *p += 1ull; break; }
        case DT_F32: { float *p = (float *)bins + b; did_overflow |= (*p == FLT_MAX); *p += 1.0f; break; }
        case DT_F64: { double *p = (double *)bins + b; did_overflow |= (*p == DBL_MAX); *p += 1.0; break; }
        default: return -1;
        }
    }
    if (overflow) *overflow |= did_overflow ? 1 : 0;
    return 0;
}

/* ------------------------------------------------------------------------------------
 * Unique: UniqueKernel (UniqueExtensions.cs:59-112): element i survives when it is the first
 * one or Compare(input[i], input[i-1]) != 0 with Comparison{T} = first.CompareTo(second)
 * (ComparisonOperations.tt); survivors are moved to the front in order.  Returns the count.
 * ---------------------------------------------------------------------------------- */
static int same_value(int dt, uint64_t a, uint64_t b) {
    if (dt == DT_F32) {
        float x, y; uint32_t ua = (uint32_t)a, ub = (uint32_t)b;
        memcpy(&x, &ua, 4); memcpy(&y, &ub, 4);
        return x == y || (x != x && y != y);
    }
    if (dt == DT_F64) {
        double x, y;
        memcpy(&x, &a, 8); memcpy(&y, &b, 8);
        return x == y || (x != x && y != y);
    }
    if (dt == DT_F16) {   /* equal bits, or +0 / -0, or both NaN */
        uint16_t x = (uint16_t)a, y = (uint16_t)b;
        int nan_x = (x & 0x7C00) == 0x7C00 && (x & 0x03FF), nan_y = (y & 0x7C00) == 0x7C00 && (y & 0x03FF);
        if (nan_x || nan_y) return nan_x && nan_y;
        return x == y || ((x | y) & 0x7FFF) == 0;
    }
    return a == b;
}

int64_t oracle_unique(int dt, void *data, int64_t n) {
    const int es = dtype_size(dt);
    uint8_t *d = (uint8_t *)data;
    int64_t out = 0;
    uint64_t prev = 0;
    for (int64_t i = 0; i < n; ++i) {
        uint64_t cur = load_raw(dt, d, i);
        if (i == 0 || !same_value(dt, cur, prev)) {
            memmove(d + out * es, d + i * es, es);
            ++out;
        }
        prev = cur;
    }
    return out;
}

/* ------------------------------------------------------------------------------------
 * Multi-core variant used only as a timed CPU baseline: the same literal two-kernel
 * radix sort, with the (independent) groups of each kernel spread over POSIX threads,
 * which is what a CPUDevice with numMultiprocessors = cores does
 * (Runtime/CPU/CPUMultiprocessor.cs:273-304 runs a multiprocessor's groups in sequence,
 * multiprocessors in parallel).  Keys only.
 * ---------------------------------------------------------------------------------- */
#include <pthread.h>

typedef struct {
    int dt, descending, num_groups, shift, phase, g0, g1;
    int64_t n, iters;
    uint8_t *k, *tmpk;
    int64_t *counter, *counter2;
} mt_job;

static void *mt_worker(void *arg) {
    mt_job *j = (mt_job *)arg;
    const int U = 4, ks = dtype_size(j->dt), dt = j->dt;
    for (int g = j->g0; g < j->g1; ++g) {
        int64_t start = (int64_t)g * j->iters, end = start + j->iters;
        int64_t maxlen = end < j->n ? end : j->n;
        if (j->phase == 1) {
            int64_t scan_mem[4] = {0, 0, 0, 0}, add_mem[4] = {0, 0, 0, 0};
            for (int64_t i = start; i < maxlen; ++i)
                ++scan_mem[oracle_extract_radix_bits(dt, load_raw(dt, j->k, i), j->shift, U - 1, j->descending)];
            for (int b = 0; b < U; ++b) j->counter[(int64_t)j->num_groups * b + g] = scan_mem[b];
            int64_t scanned = 0, previous = scan_mem[0];
            for (int b = 1; b < U; ++b) { scanned += previous; previous = scan_mem[b]; scan_mem[b] = scanned; }
            scan_mem[0] = 0;
            for (int64_t i = start; i < maxlen; ++i) {
                int b = oracle_extract_radix_bits(dt, load_raw(dt, j->k, i), j->shift, U - 1, j->descending);
                int64_t pos = start + add_mem[b]++ + scan_mem[b];
                memcpy(j->tmpk + pos * ks, j->k + i * ks, ks);
            }
        } else {
            for (int64_t i = start; i < maxlen; ++i) {
                int b = oracle_extract_radix_bits(dt, load_raw(dt, j->tmpk, i), j->shift, U - 1, j->descending);
                int64_t idx = (int64_t)b * j->num_groups + g;
                int64_t pos = (idx < 1 ? 0 : j->counter2[idx - 1]) + i - start;
                int64_t offset = 0;
                for (int w = 0; w < b; ++w) {
                    int64_t a = (int64_t)w * j->num_groups + g;
                    offset += j->counter2[a] - (a < 1 ? 0 : j->counter2[a - 1]);
                }
                pos -= offset;
                memcpy(j->k + pos * ks, j->tmpk + i * ks, ks);
            }
        }
    }
    return NULL;
}

int oracle_radix_sort_literal_mt(int dt, void *keys, int64_t n, int descending, int num_groups,
                                 int num_threads) {
    if (n <= 0) return 0;
    if (num_threads < 1) num_threads = 1;
    if (num_threads > num_groups) num_threads = num_groups;
    const int U = 4, bit_inc = 2, ks = dtype_size(dt);
    int64_t iters = (n + num_groups - 1) / num_groups;
    uint8_t *tmpk = (uint8_t *)malloc((size_t)n * ks);
    int64_t *counter = (int64_t *)calloc((size_t)num_groups * U, sizeof(int64_t));
    int64_t *counter2 = (int64_t *)calloc((size_t)num_groups * U, sizeof(int64_t));
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)num_threads);
    mt_job *jobs = (mt_job *)malloc(sizeof(mt_job) * (size_t)num_threads);
    for (int shift = 0; shift < ks * 8; shift += bit_inc) {
        for (int phase = 1; phase <= 2; ++phase) {
            for (int t = 0; t < num_threads; ++t) {
                mt_job j = {dt, descending, num_groups, shift, phase,
                            (int)((int64_t)num_groups * t / num_threads),
                            (int)((int64_t)num_groups * (t + 1) / num_threads),
                            n, iters, (uint8_t *)keys, tmpk, counter, counter2};
                jobs[t] = j;
                pthread_create(&th[t], NULL, mt_worker, &jobs[t]);
            }
            for (int t = 0; t < num_threads; ++t) pthread_join(th[t], NULL);
            if (phase == 1) {
                int64_t run = 0;
                for (int64_t i = 0; i < (int64_t)num_groups * U; ++i) { run += counter[i]; counter2[i] = run; }
            }
        }
    }
    free(tmpk); free(counter); free(counter2); free(th); free(jobs);
    return 0;
}
