/*
 * homura_cuda_shard.h: reductions of a tensor that is split along its outermost dimension over the
 * GPUs of one machine.
 *
 * homura has no multi-GPU collective of any kind (its devices exchange data through host memory, one
 * device lock at a time, src/backend/mod.rs:240-255), so nothing here replaces a declaration of
 * csrc/homura_rocm.h; this is the exchange step its reductions need once a tensor is sharded. Elementwise
 * work, reductions over inner dimensions and softmax over the last dimension need no exchange at all:
 * each GPU runs the ordinary entry points on its shard.
 *
 * A reduction that folds the sharded dimension runs in three steps, all on the contexts' streams:
 *   1. every rank folds its shard into per-output partials that keep the accumulator's precision
 *      (f64 for float sums, products and means: hmc_reduce_partial; integer sums, max/min values and
 *      their indices, and the 0/1 results of all / any are exact already and come from hmc_reduce /
 *      hmc_arg_reduce; all / any combine as the minimum / maximum of the ranks' results);
 *   2. the partials of all ranks are gathered into every rank's own memory (hmc_comm_allgather: one NCCL
 *      all-gather of a few bytes per output, latency bound);
 *   3. every rank folds the gathered partials in rank order (hmc_shard_combine_*): the same bits on every
 *      rank and on every run, "first NaN, then first of equals" across shards as within one, and global
 *      indices for the arg reductions. (An NCCL all-reduce with ncclSum / ncclMax promises neither an
 *      order nor a NaN rule, which is why the combine is a kernel of this library.)
 *
 * The hmc_comm_* entry points live in libhomura_cuda_shard.so, which links NCCL; the rest is in
 * libhomura_cuda.so.
 */
#ifndef HOMURA_CUDA_SHARD_H
#define HOMURA_CUDA_SHARD_H

#include "homura_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* hmc_reduce for float SUM, PROD or MEAN that stops before the rounding: partial[o] is the f64 sum (or
 * product) of output o's elements on this shard (MEAN gives the sum). `partial` holds one f64 per output
 * in device memory. Workspace as for hmc_reduce. */
hmc_status hmc_reduce_partial(hmc_context_t ctx, int32_t op, double *partial, const hmc_tensor_desc *kept,
                              const hmc_tensor_desc *red, void *workspace, int64_t workspace_bytes);

/* out[o] = round(fold over r = 0..ranks-1 of gathered[r * nout + o]) for SUM and PROD, the sum divided by
 * total_count for MEAN. `out` is a contiguous float tensor of nout elements. */
hmc_status hmc_shard_combine_float(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const double *gathered,
                                   int32_t ranks, int64_t nout, int64_t total_count);

/* Wrapping i64 SUM or PROD of the ranks' I64 results. */
hmc_status hmc_shard_combine_int(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const int64_t *gathered,
                                 int32_t ranks, int64_t nout);

/* Maximum or minimum over the ranks' results: gathered_values[r * nout + o] has the dtype of out_values;
 * gathered_indices (may be NULL) holds each rank's local index along the sharded dimension, to which
 * index_offsets[r] (host memory, `ranks` entries: the first global index of rank r's shard) is added.
 * A NaN of the lowest rank wins, then the first of equal values. Either output may be NULL. */
hmc_status hmc_shard_combine_extreme(hmc_context_t ctx, int32_t is_max, const hmc_tensor_desc *out_values,
                                     const hmc_tensor_desc *out_indices, const void *gathered_values, int32_t dtype,
                                     const int64_t *gathered_indices, const int64_t *index_offsets, int32_t ranks,
                                     int64_t nout);

/* Variance / standard deviation across shards, two rounds as on one GPU (cpu::var, src/backend/cpu/reduce.rs:135-170:
 * the mean in f64, then the squared deviations from it):
 *   first exchange: hmc_reduce_partial(SUM) -> all-gather -> hmc_shard_combine_means: means[o] = (sum over the ranks in
 *            rank order) / total_count, kept in f64 (one per output, device memory);
 *   second exchange: hmc_var_partial: partial[o] = the f64 sum over this shard of (x - means[o])^2 (workspace as for
 *            hmc_reduce) -> all-gather -> hmc_shard_combine_var: out[o] = round(sum over the ranks / (total_count -
 *            correction)), its square root with take_sqrt, NaN when total_count is 0, infinity or NaN when the
 *            divisor is not positive (as hmc_var). */
hmc_status hmc_shard_combine_means(hmc_context_t ctx, double *means, const double *gathered, int32_t ranks, int64_t nout,
                                   int64_t total_count);
hmc_status hmc_var_partial(hmc_context_t ctx, double *partial, const hmc_tensor_desc *kept, const hmc_tensor_desc *red,
                           const double *means, void *workspace, int64_t workspace_bytes);
hmc_status hmc_shard_combine_var(hmc_context_t ctx, const hmc_tensor_desc *out, const double *gathered, int32_t ranks,
                                 int64_t nout, int64_t total_count, double correction, int32_t take_sqrt);

/* ---- NCCL (libhomura_cuda_shard.so) ---- */
#define HMC_COMM_ID_BYTES 128
typedef struct hmc_comm *hmc_comm_t;

/* A fresh identifier for a communicator; rank 0 makes it and hands it to the others by any channel. */
hmc_status hmc_comm_unique_id(uint8_t *id);
/* Joins the communicator `id` as `rank` of `ranks` with the context's device and stream (collective:
 * every rank calls it). The communicator never blocks a caller for ever: every call gives the library at most
 * the communicator's timeout (60 s unless the environment variable HMC_COMM_TIMEOUT_MS or hmc_comm_set_timeout
 * says otherwise) to make progress. When the time runs out, or the library reports an error of an earlier
 * collective, the communicator is aborted (kernels of it that still wait for a peer stop; the context and its
 * stream stay usable), the call returns HMC_CUDA_ERROR and every later call on the communicator HMC_INVALID. */
hmc_status hmc_comm_create(hmc_context_t ctx, int32_t ranks, int32_t rank, const uint8_t *id, hmc_comm_t *out);
hmc_status hmc_comm_set_timeout(hmc_comm_t comm, int64_t milliseconds);
hmc_status hmc_comm_destroy(hmc_comm_t comm);
/* Queues an all-gather on the context's stream: rank r's `bytes` bytes at `send` land at
 * recv + r * bytes on every rank. send and recv are device memory of the context's device. */
hmc_status hmc_comm_allgather(hmc_comm_t comm, const void *send, void *recv, uint64_t bytes);
/* Waits, for at most the timeout, until everything queued on the context's stream has run (the collectives
 * included). Where hmc_context_synchronize would wait for ever on a collective whose peer never joined, this
 * aborts the communicator and returns HMC_CUDA_ERROR. */
hmc_status hmc_comm_wait(hmc_comm_t comm);
/* Tears the communicator down without the peers (which hmc_comm_destroy's orderly shutdown expects to be there):
 * for a rank that has learnt that a peer is gone. hmc_comm_destroy still frees the handle afterwards. */
hmc_status hmc_comm_abort(hmc_comm_t comm);

#ifdef __cplusplus
}
#endif

#endif /* HOMURA_CUDA_SHARD_H */
