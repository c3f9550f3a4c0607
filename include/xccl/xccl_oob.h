/*
 * xccl-b200: ready-made out-of-band providers (extension; the reference leaves the OOB
 * allgather to its caller and its tests build one on MPI, test/test_mpi.c:19-97).
 *
 * Shared-memory provider: all ranks live on one host and agree on a job key. Every pair of
 * ranks owns a small mailbox in a POSIX shared-memory segment; an allgather over any group
 * (whole job or an endpoint range) is N-1 mailbox writes and N-1 mailbox reads driven by
 * req_test(), so it never blocks and needs no helper thread.
 */
#ifndef XCCL_B200_OOB_H_
#define XCCL_B200_OOB_H_

#include "xccl.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Fills *oob (functions, coll_context, rank, size). job_key must be unique per job: a stale
 * segment of a crashed job with the same key would be reused. Rank order is the caller's. */
xccl_status_t xccl_oob_shm_create(const char *job_key, int rank, int size, xccl_oob_collectives_t *oob);
/* Detaches; the last rank to leave removes the segment. */
void          xccl_oob_shm_destroy(xccl_oob_collectives_t *oob);

/* A view of `parent` restricted to `n` of its ranks (parent_ranks[i] = parent rank of member
 * i). The caller must be one of them. Used to bootstrap sub-teams. Free with
 * xccl_oob_sub_destroy. */
xccl_status_t xccl_oob_sub_create(const xccl_oob_collectives_t *parent, const int *parent_ranks, int n,
                                  xccl_oob_collectives_t *sub);
void          xccl_oob_sub_destroy(xccl_oob_collectives_t *sub);

/* Blocking allgather over a provider with the XCCL_OOB_TIMEOUT deadline. */
xccl_status_t xccl_oob_allgather(const xccl_oob_collectives_t *oob, void *sbuf, void *rbuf, size_t size);

#ifdef __cplusplus
}
#endif

#endif
