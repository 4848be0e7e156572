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

#ifdef __cplusplus
}
#endif
#endif /* B200ALG_TESTING_H */
