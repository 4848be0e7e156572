/*
 * b200alg - entry points for the test-suite only; not part of the product ABI (no binding
 * in the host mirrors, no stability promise).
 */
#ifndef B200ALG_TESTING_H
#define B200ALG_TESTING_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Launches one warp that polls a word of `temp` which nothing ever sets, with the bounded
 * wait the product kernels use for their look-back, limited to max_polls (<= 10^6) polls.
 * The wait runs out, the kernel records that in temp's control block and returns; the
 * context stays usable.  b200alg_device_status(stream, temp) then reports
 * B200ALG_WAIT_LIMIT.  temp: at least 512 bytes, 256-byte aligned. */
int b200alg_testing_wait_limit(void *stream, void *temp, int64_t temp_bytes, unsigned int max_polls);

/* b200alg_radix_sort_keys (dense view) with CUDA events around digit pass `pass` (0 = least
 * significant byte) on `stream`; synchronises the stream and returns the pass's device time.
 * The sort call is one entry point, so a caller cannot bracket a single pass by itself; the
 * benchmark uses this for the roofline figure of the digit-pass kernel.  A pass whose digit is
 * constant over all keys exits at once and reads as a few microseconds. */
int b200alg_testing_time_sort_pass(void *stream, void *keys, int64_t n, int key_dtype, int order, void *temp,
                                   int64_t temp_bytes, int pass, float *milliseconds);

/* Exported by libb200alg_mg.so.  b200alg_sort_mg (include/b200alg_mg.h: same arguments, comm is a
 * b200alg_comm*, collective over the ranks) with CUDA events where its phases meet; synchronises
 * the stream and returns the device time of this rank's six phases in phase_ms[0..6): splitters
 * (samples into the mailboxes, barrier, selection), bucket sizes (count, row into the
 * mailboxes), barrier and the plan of the exchange, partition with peer stores, last barrier
 * (the wait for the slowest sender), local sort. */
int b200alg_testing_time_sort_mg(void *comm, void *stream, const void *keys, const void *values, int64_t n,
                                 int key_dtype, int value_bytes, int order, void *out_keys, void *out_values,
                                 int64_t out_capacity, int64_t *out_count, float *phase_ms);

#ifdef __cplusplus
}
#endif
#endif /* B200ALG_TESTING_H */
