/*
 * Row-sharded f64 GEMM over the GPUs of one box, for a C host (one process per GPU).
 *
 * The reference is single-device; this is the multi-GPU form of its exact tier
 * (ozaki_ii_dispatch, lib/backend/gpu/gpu_memory.mm:2474-2771): rows of A are independent in
 * that tier, so rank r multiplies rows [row0_r, row0_r + rows_r) of A by B and every rank ends
 * up with the whole C, bit for bit the product one GPU would give.  B lives on one rank; every
 * rank scans and splits 1/world of each column panel of B and the ranks exchange the residue
 * planes, and the blocks of C, with copy-engine transfers over NVLink (CUDA IPC mappings and
 * interprocess events).  No collective library is involved: the ranks find each other through
 * a named POSIX shared-memory segment, which also carries the host barriers.
 *
 * Every process calls eshkol_b200_init(device) first, then the same sequence of calls here
 * with the same arguments.  All functions return 0, or -1 after writing one line to stderr;
 * a rank that fails marks the session failed, and the other ranks' barriers then return -1
 * instead of waiting (their own timeout is 60 seconds).
 */
#ifndef ESHKOL_B200_MULTI_H
#define ESHKOL_B200_MULTI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct EshkolB200Sharded EshkolB200Sharded;

/* Joins (rank 0: creates) the session `name` -- a shared-memory name such as "/eshkol-1234",
 * fresh for every session -- of `world` ranks (at most 16) for products of shape M x K x N with
 * K <= 262144, allocates this rank's buffers and opens the peers'.  src_rank is the rank that
 * holds B.  Collective: returns on every rank when all have joined. */
int eshkol_b200_sharded_open(const char* name, int rank, int world, uint64_t M, uint64_t K, uint64_t N,
                             int src_rank, EshkolB200Sharded** out);

/* This rank's block of rows. */
int eshkol_b200_sharded_rows(const EshkolB200Sharded* s, uint64_t* row0, uint64_t* rows);

/* Device memory of the session: on src_rank the K x N matrix B is read from b_buffer (the
 * caller fills it, on any stream it has synchronised, before a step); c_buffer is the M x N
 * result, complete on every rank when a step returns.  b_buffer is NULL on the other ranks. */
double* eshkol_b200_sharded_b_buffer(EshkolB200Sharded* s);
double* eshkol_b200_sharded_c_buffer(EshkolB200Sharded* s);

/* One product.  dA_rows: this rank's rows of A (rows x K, device memory, complete before the
 * call).  Collective; returns when this rank's C is complete and no peer still reads a buffer
 * of this rank. */
int eshkol_b200_sharded_step(EshkolB200Sharded* s, const double* dA_rows);

/* Collective.  Closes the peers' mappings, frees this rank's buffers; rank 0 unlinks the name. */
int eshkol_b200_sharded_close(EshkolB200Sharded* s);

#ifdef __cplusplus
}
#endif

#endif /* ESHKOL_B200_MULTI_H */
