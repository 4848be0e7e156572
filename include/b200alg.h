/*
 * b200alg - data-parallel primitives (radix sort, scan, reduce, histogram) for NVIDIA
 * B200 (sm_100a) behind the ILGPU.Algorithms API.
 *
 * C ABI: plain pointers and sizes only.  Every pointer named `stream` is a CUstream /
 * cudaStream_t (NULL = the legacy default stream); every data pointer is a device
 * address in the CUDA context that is current on the calling thread.  All work is
 * enqueued on `stream`; no function synchronises with the host unless its comment says
 * so.  The library allocates no device memory: scratch space comes from the caller
 * (`temp`, sized by the *_temp_bytes helpers).  No pointer is retained after return.
 * Concurrent calls are legal only with distinct temp buffers.
 *
 * Each entry point cites the ILGPU item it replaces (file:line inside the ILGPU source
 * tree, Src/ILGPU.Algorithms unless another directory is given).
 */
#ifndef B200ALG_H
#define B200ALG_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200ALG_VERSION 100 /* major*10000 + minor*100 + patch */

/* Element types.  Sort keys accept all of them (the 11 key types of
 * RadixSortOperations.tt:26-125); scan / reduce / histogram accept the six "atomic
 * numeric types" I32, U32, I64, U64, F32, F64 (ScanReduceOperations.tt:20-74,
 * HistogramOperations.tt:30-41). */
typedef enum {
    B200ALG_I8 = 0, B200ALG_U8 = 1, B200ALG_I16 = 2, B200ALG_U16 = 3,
    B200ALG_I32 = 4, B200ALG_U32 = 5, B200ALG_I64 = 6, B200ALG_U64 = 7,
    B200ALG_F16 = 8, B200ALG_F32 = 9, B200ALG_F64 = 10
} b200alg_dtype;

/* Scan / reduce operations: Add*, Max*, Min* of ScanReduceOperations.tt:20-26. */
typedef enum { B200ALG_ADD = 0, B200ALG_MAX = 1, B200ALG_MIN = 2 } b200alg_op;

/* Sort order flags.  DESCENDING selects the Descending* structs
 * (RadixSortOperations.tt:100-125).  FLOAT_TOTAL_ORDER is an opt-in that orders
 * F16/F32/F64 keys numerically (IEEE total order); without it float keys follow the
 * reference's ExtractRadixBits literally (RadixSortOperations.tt:81-89). */
#define B200ALG_SORT_ASCENDING 0
#define B200ALG_SORT_DESCENDING 1
#define B200ALG_SORT_FLOAT_TOTAL_ORDER 2

/* Named histogram bin locators (the reference leaves IComputeSingleBinOperation to user
 * structs, IHistogramOperations.cs:19-78; a C ABI needs a closed set).
 *  EQUAL_WIDTH_CLAMP: t = (x - lo) * (num_bins / (hi - lo)) with the scale computed once
 *      in the input's floating type (double for integer inputs); bin = floor(t) clamped
 *      to [0, num_bins-1]; NaN -> bin 0.  hi > lo must also hold, and the scale be finite,
 *      in that type (B200ALG_INVALID_ARGUMENT otherwise).
 *  MODULO: the reference tests' ModuloBin*Operation (ILGPU.Algorithms.Tests/
 *      HistogramTests.tt:83-94): |x % num_bins| for integers, (int)|fmod(x, num_bins)|
 *      for floats. */
typedef enum { B200ALG_LOCATOR_EQUAL_WIDTH_CLAMP = 0, B200ALG_LOCATOR_MODULO = 1 } b200alg_locator;

typedef enum {
    B200ALG_OK = 0,
    B200ALG_INVALID_ARGUMENT = 1,   /* null pointer, negative size, bad stride */
    B200ALG_UNSUPPORTED = 2,        /* dtype / op / value size outside the closed set */
    B200ALG_TEMP_TOO_SMALL = 3,
    B200ALG_CUDA_ERROR = 4,         /* see b200alg_last_cuda_error() */
    B200ALG_WAIT_LIMIT = 5,         /* a device-side wait ran out (reported by b200alg_device_status) */
    B200ALG_MISALIGNED = 6,         /* a pointer is not aligned to its element size / temp not to 256 */
    B200ALG_TOO_LARGE = 7,          /* n beyond 2^38; the int.MaxValue limit of the reference (ErrorMessages.NotSupportedArrayView64) is the host mirror's check */
    B200ALG_STATIC_LIMIT = 8,       /* n beyond what an entry point with built-in scratch accepts */
    B200ALG_NCCL_ERROR = 9          /* multi-GPU layer (b200alg_mg.h): a NCCL call failed */
} b200alg_status;

int b200alg_version(void);
const char *b200alg_status_string(int status);
/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
int b200alg_last_cuda_error(void);

/* ---- radix sort -------------------------------------------------------------------
 * Replaces the lambdas returned by CreateRadixSort (RadixSortExtensions.cs:1130-1337)
 * and CreateRadixSortPairs (:1017-1118).  In place, LSD, stable.  `order` is a bit-or of
 * the B200ALG_SORT_* flags. */

/* Native counterpart of ComputeRadixSortTempStorageSize (:419-447) and
 * ComputeRadixSortPairsTempStorageSize (:384-404); result in bytes (a multiple of 256).
 * value_bytes = 0 for keys only. */
int b200alg_radix_sort_temp_bytes(int key_dtype, int64_t n, int value_bytes, int64_t *out_bytes);

/* keys: n elements `stride` elements apart (ArrayView1D<T, TStride>; dense = 1). */
int b200alg_radix_sort_keys(void *stream, void *keys, int64_t n, int64_t stride, int key_dtype,
                            int order, void *temp, int64_t temp_bytes);

/* values: n dense elements of value_bytes (1, 2, 4, 8 or 16) each, permuted like the keys. */
int b200alg_radix_sort_pairs(void *stream, void *keys, void *values, int64_t n, int key_dtype,
                             int value_bytes, int order, void *temp, int64_t temp_bytes);

/* The sequencer overload of CreateRadixSortPairs (RadixSortExtensions.cs:1017-1074, gather
 * kernel :605-625): the values that enter the sort are not read from `values` but made
 * from the element index by one of the reference's built-in sequencers - (T)i for the
 * integer types (IndexSequencer, Sequencer.cs:37-42; {Int8..UInt64}Sequencer,
 * Sequencers.tt:26-38), the converted index for F16 / F32 / F64 (Half-, Float-,
 * DoubleSequencer, Sequencer.cs:47-72) - inside the first digit pass, so "payload =
 * original index" costs neither a fill pass nor a read of the value view.  `values`
 * (n dense elements of value_dtype) only receives the permuted result.  Temp size: that of
 * b200alg_radix_sort_temp_bytes with value_bytes = the size of value_dtype. */
int b200alg_radix_sort_pairs_sequence(void *stream, void *keys, void *values, int64_t n, int key_dtype,
                                      int value_dtype, int order, void *temp, int64_t temp_bytes);

/* The same sort out of place: in_keys / in_values are only read, the result lands in
 * out_keys / out_values (dense views, distinct from the inputs).  No counterpart in the
 * reference (its sorts are in place); the last step of a sort that spans several GPUs uses
 * it to sort straight out of its receive buffer.  n_device, when not NULL, points to the
 * element count in device memory (int64): n is then only an upper bound that sizes temp and
 * the launches, and nothing beyond *n_device elements is read or written - the count may
 * still be produced by earlier work on the same stream when this call is enqueued. */
int b200alg_radix_sort_out_of_place(void *stream, const void *in_keys, const void *in_values, void *out_keys,
                                    void *out_values, int64_t n, const int64_t *n_device, int key_dtype,
                                    int value_bytes, int order, void *temp, int64_t temp_bytes);

/* Stable partition of a shard into num_splitters + 1 buckets: the first step of a sort
 * that spans several GPUs (new surface; the reference has no multi-device sort, its only
 * multi-GPU facility is peer access, Src/ILGPU/Runtime/PeerAccess.cs).  Element i goes to
 * bucket #{s : (splitter_keys[s], splitter_index[s]) <= (keys[i], index_base + i)} in the
 * order (transformed key, index); inside a bucket the input order is kept.  out_keys /
 * out_values receive the buckets one after the other, bucket_counts (int64, device) their
 * sizes.  Splitters are device arrays and must be ascending in that order.
 * value_bytes in {0, 4, 8}. */
int b200alg_bucket_partition_temp_bytes(int key_dtype, int64_t n, int64_t *out_bytes);
int b200alg_bucket_partition(void *stream, const void *keys, const void *values, int64_t n, int key_dtype,
                             int value_bytes, int order, const void *splitter_keys,
                             const int64_t *splitter_index, int num_splitters, int64_t index_base,
                             void *out_keys, void *out_values, int64_t *bucket_counts, void *temp,
                             int64_t temp_bytes);

/* The same partition in two steps, for a sort whose exchange is fused into the partition:
 * b200alg_bucket_count only sizes the buckets; after the ranks have exchanged the sizes,
 * b200alg_bucket_scatter stores bucket b of this shard at bucket_key_ptrs[b][0..count_b)
 * (and bucket_value_ptrs[b][...]), in input order.  The pointer tables are device arrays
 * of num_splitters + 1 entries; an entry may point into another GPU's memory that is
 * mapped into this process (the stores then travel over NVLink; plain stores, no TMA). */
int b200alg_bucket_count(void *stream, const void *keys, int64_t n, int key_dtype, int order,
                         const void *splitter_keys, const int64_t *splitter_index, int num_splitters,
                         int64_t index_base, int64_t *bucket_counts, void *temp, int64_t temp_bytes);
int b200alg_bucket_scatter(void *stream, const void *keys, const void *values, int64_t n, int key_dtype,
                           int value_bytes, int order, const void *splitter_keys,
                           const int64_t *splitter_index, int num_splitters, int64_t index_base,
                           void *const *bucket_key_ptrs, void *const *bucket_value_ptrs, void *temp,
                           int64_t temp_bytes);

/* Splitters out of a sample of (key, index) pairs without sorting it: for j in [0, num_picks)
 * the pair of rank ((j + 1) * m) / (num_picks + 1) in the order a stable sort of the keys with
 * `order` would give (equal keys keep their slot order), raw key bits and index.  m is read on
 * the device from m_device[0] and clamped to [0, max_m]; m == 0 yields zeros.  Every pair counts
 * the pairs in front of it (quadratic: max_m <= 65536).  temp: max_m * 4 bytes, 4-byte aligned.
 * No counterpart in the reference; the multi-GPU sort picks its splitters with it. */
int b200alg_select_splitters(void *stream, const void *keys, const int64_t *index, int64_t max_m,
                             const int64_t *m_device, int key_dtype, int order, int num_picks,
                             void *out_keys, int64_t *out_index, void *temp, int64_t temp_bytes);

/* ---- scan -------------------------------------------------------------------------
 * Replaces the lambda of CreateScan (ScanExtensions.cs:930-959 -> SinglePassScanKernel
 * :530-706).  out[i*out_stride] = fold(op, in[0..i]) (inclusive) or fold(op, in[0..i-1])
 * with out[0] = Identity (exclusive).  in == out is allowed when the strides match. */
int b200alg_scan_temp_bytes(int dtype, int64_t n, int64_t *out_bytes); /* ComputeScanTempStorageSize :158-170 */
int b200alg_scan(void *stream, const void *in, int64_t in_stride, void *out, int64_t out_stride,
                 int64_t n, int dtype, int op, int inclusive, void *temp, int64_t temp_bytes);
/* Same, with the running value that precedes in[0] read from device memory
 * (`carry_in`, one element, may be NULL = Identity): what a sharded scan uses to add
 * the total of the lower ranks.  New surface; the reference has no multi-device scan. */
int b200alg_scan_carry(void *stream, const void *in, int64_t in_stride, void *out, int64_t out_stride,
                       int64_t n, int dtype, int op, int inclusive, const void *carry_in,
                       void *temp, int64_t temp_bytes);

/* Scan for callers that cannot hand over a temp view.  No counterpart in the reference:
 * there every scan takes (or, through ScanProvider, owns) a temp buffer.  This variant is
 * for code that gets an input and an output view and has no way to allocate - a stream
 * callback, a loop that must not touch the allocator, a host that forbids cudaMalloc after
 * start-up.  The tile descriptors live in an array built into the library (about 2 MiB of
 * device memory on every GPU that loads it, held until the process exits), which
 * limits n to 2^26 elements (B200ALG_STATIC_LIMIT beyond that).  The call allocates
 * nothing.  The first call on each device looks up the array's device address; make that
 * first call outside any stream capture.  All calls on one device share the array: two
 * calls whose kernels may overlap on the GPU (different streams) corrupt each other;
 * calls on the same stream are fine, each one clears what it uses. */
#define B200ALG_SCAN_STATIC_MAX_ELEMENTS (1ll << 26)
int b200alg_scan_static(void *stream, const void *in, int64_t in_stride, void *out, int64_t out_stride,
                        int64_t n, int dtype, int op, int inclusive);

/* ---- reduce -----------------------------------------------------------------------
 * Replaces the lambda of CreateReduction (ReductionExtensions.cs:135-167): out[0] is set
 * to Identity and then folded with every input element.  n >= 1. */
int b200alg_reduce(void *stream, const void *in, int64_t stride, int64_t n, int dtype, int op, void *out);

/* ---- histogram --------------------------------------------------------------------
 * Replaces the lambdas of CreateHistogram / CreateHistogramUnchecked
 * (HistogramExtensions.cs:293-354, :371-427) with the single-bin adapter
 * (HistogramLaunchers.tt:52-101).  bins[locator(x)] += 1 for every element; bins are
 * accumulated into, never cleared.  overflow (int32[1], may be NULL = unchecked variant)
 * gets |= 1 when an increment started from the bin type's MaxValue
 * (HistogramOperations.tt:36-40). */
int b200alg_histogram(void *stream, const void *in, int64_t stride, int64_t n, int in_dtype,
                      int locator, double lo, double hi, void *bins, int64_t num_bins, int bin_dtype,
                      void *overflow);

/* ---- helpers on the path's edges --------------------------------------------------- */
/* InitializeExtensions.cs (CreateInitializer): view[i*stride] = *value (elem_bytes bytes, host pointer). */
int b200alg_initialize(void *stream, void *view, int64_t stride, int64_t n, int elem_bytes, const void *value);
/* SequenceExtensions.cs with the Int32/Int64/UInt32/UInt64 sequencers of Sequencers.tt:
 * view[i] = (T)(start + i * step); dtype in {I32, U32, I64, U64}. */
int b200alg_sequence(void *stream, void *view, int64_t n, int dtype, int64_t start, int64_t step);

/* UniqueExtensions.cs:59-195 (CreateUnique with the Comparison{T} operations of
 * ComparisonOperations.tt): removes consecutive duplicates of data[0..n) in place and stores
 * the number of elements left in out_count[0] (int64, device).  Integers compare by value;
 * floating-point values are equal when numerically equal or both NaN (CompareTo).  temp
 * holds the survivors before they are copied back, so it grows with n (the reference's
 * ComputeUniqueTempStorageSize is one int because its kernel is a serial chain of groups). */
int b200alg_unique_temp_bytes(int dtype, int64_t n, int64_t *out_bytes);
int b200alg_unique(void *stream, void *data, int64_t n, int dtype, void *out_count, void *temp, int64_t temp_bytes);

/* Run-length encoding: the step after a sort when the counts per key are wanted (sort ->
 * unique -> counts).  values[r] = the element that starts run r of data[0..n), lengths[r]
 * (int64) = how many consecutive equal elements it has, num_runs[0] (int64, device) = the
 * number of runs; `data` is only read; values and lengths need room for n entries in the
 * worst case.  Equality as in b200alg_unique.  No counterpart in the reference (its
 * UniqueExtensions drop the duplicates without counting them). */
int b200alg_run_length_encode_temp_bytes(int dtype, int64_t n, int64_t *out_bytes);
int b200alg_run_length_encode(void *stream, const void *data, int64_t n, int dtype, void *values, int64_t *lengths,
                              int64_t *num_runs, void *temp, int64_t temp_bytes);

/* Device-side waits (decoupled look-back) are bounded; when one runs out the kernel
 * records it in `temp` and finishes.  This call copies that record back and
 * SYNCHRONISES `stream`: returns B200ALG_OK or B200ALG_WAIT_LIMIT. */
int b200alg_device_status(void *stream, const void *temp);

#ifdef __cplusplus
}
#endif
#endif /* B200ALG_H */
