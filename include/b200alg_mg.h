/*
 * b200alg_mg - the same primitives over the GPUs of one box (libb200alg_mg.so; needs
 * libb200alg.so and NCCL).
 *
 * The reference has no multi-device algorithms (its only multi-GPU facility is peer access,
 * Src/ILGPU/Runtime/PeerAccess.cs), so everything here is new surface.  One communicator per
 * GPU ("rank"); every rank calls the same entry point with its shard, on its own stream.
 * Ranks may be separate processes (b200alg_comm_create_rank, one GPU per process) or host
 * threads of one process (b200alg_comm_create, what a host with several accelerators in
 * one process - ILGPU's model - would use; every rank's call must then come from its own
 * thread, as with NCCL).  Data of rank r precedes data of rank r + 1 in every ordering
 * the primitives define.
 *
 * Exchange steps: reduce, histogram and scan use an NCCL all-reduce / all-gather of a few
 * words on the caller's stream.  The sort exchanges everything with plain stores into peer
 * memory over NVLink (no TMA, no multicast) between barriers of the library's own: its
 * samples and bucket sizes go into mailboxes that every rank maps, its buckets from the
 * partition kernel straight into the owner's receive buffer.  Waits between GPUs are NCCL's
 * or bounded polls that end in B200ALG_WAIT_LIMIT (b200alg_comm_status).
 */
#ifndef B200ALG_MG_H
#define B200ALG_MG_H

#include <stdint.h>

#include "b200alg.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200alg_comm b200alg_comm;

#define B200ALG_UNIQUE_ID_BYTES 128

/* Rendezvous token: made by one rank, handed to all others by whatever means the host has. */
int b200alg_comm_unique_id(void *id_bytes);

/* One GPU per caller: joins rank `rank` of `num_ranks` with the device that is current on the
 * calling thread.  Collective (returns when every rank has joined).  sort_capacity = the
 * largest number of elements a rank may receive in b200alg_sort_mg (0: the sort is not
 * used); the communicator allocates its receive buffer and sort scratch once, here. */
int b200alg_comm_create_rank(const void *id_bytes, int num_ranks, int rank, int64_t sort_capacity, b200alg_comm **out);

/* All ranks in one process: devices devs[0..ndev), out[0..ndev).  Afterwards rank i's calls
 * must come from a host thread of their own (every call is a collective). */
int b200alg_comm_create(int ndev, const int *devs, int64_t sort_capacity, b200alg_comm **out);

int b200alg_comm_destroy(b200alg_comm *comm);
int b200alg_comm_rank(const b200alg_comm *comm, int *rank, int *num_ranks);
/* Synchronises `stream`; B200ALG_WAIT_LIMIT if a bounded wait between GPUs ran out or the
 * sort's receive buffer was too small since the last query (the flag is cleared). */
int b200alg_comm_status(b200alg_comm *comm, void *stream);
int b200alg_comm_last_nccl_error(const b200alg_comm *comm);

/* out[0] (on every rank) = fold of all ranks' inputs.  Integers bit-exact; floating-point
 * sums differ from a single-GPU run by the usual reassociation. */
int b200alg_reduce_mg(b200alg_comm *comm, void *stream, const void *in, int64_t stride, int64_t n, int dtype, int op,
                      void *out);

/* bins (replicated: every rank passes bins of equal content) += the counts of all ranks'
 * inputs; overflow as in b200alg_histogram, decided on the summed counts. */
int b200alg_histogram_mg(b200alg_comm *comm, void *stream, const void *in, int64_t stride, int64_t n, int in_dtype,
                         int locator, double lo, double hi, void *bins, int64_t num_bins, int bin_dtype, void *overflow);

/* Scan of the concatenation of the ranks' inputs in rank order; every rank writes its
 * slice.  Dense views.  temp as for b200alg_scan. */
int b200alg_scan_mg(b200alg_comm *comm, void *stream, const void *in, void *out, int64_t n, int dtype, int op,
                    int inclusive, void *temp, int64_t temp_bytes);

/* Sample sort.  Rank r ends up with the r-th slice of the sorted whole in out_keys /
 * out_values (capacity out_capacity elements) and its length in out_count[0] (int64, device
 * memory).  Stable: equal keys keep the order (rank, position) they had on entry.  keys /
 * values are only read.  value_bytes in {0, 4, 8}.  No host synchronisation: the slice length
 * is never needed on the host. */
int b200alg_sort_mg(b200alg_comm *comm, void *stream, const void *keys, const void *values, int64_t n, int key_dtype,
                    int value_bytes, int order, void *out_keys, void *out_values, int64_t out_capacity,
                    int64_t *out_count);

#ifdef __cplusplus
}
#endif
#endif /* B200ALG_MG_H */
