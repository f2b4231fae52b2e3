/* tagi_b200_comm.h - C ABI of the data-parallel exchange of TAGI parameter deltas (libtagi_b200_comm.so).
 *
 * Replaces NCCLCommunicator and DDPSequential::sync_parameters / sync_base_parameters (src/ddp.cpp:27-72, 113-177,
 * include/ddp.h:26-145 of cuTAGI): one process per GPU, every rank holds a full parameter replica, and before `step`
 * the parameter deltas (delta_mu_w, delta_var_w, delta_mu_b, delta_var_b of every layer) are averaged or summed over
 * the ranks. Differences from the reference, by design:
 *   - no MPI: the ncclUniqueId travels through a rendezvous file (or any channel of the caller's);
 *   - tensors are registered once, in the order their backward passes finish, and grouped into buckets of a byte
 *     budget; one bucket = one fused NCCL launch (ncclGroupStart / ncclGroupEnd);
 *   - a bucket is launched on a private communication stream as soon as its last tensor has been produced (an event on
 *     the compute stream orders it), so it overlaps the backward pass of the layers below; `step` waits with
 *     tagi_comm_wait, which is a stream wait, not a host synchronisation;
 *   - nested layers are the caller's to enumerate: whatever is registered is exchanged (the reference walks only the
 *     top-level layer list and skips everything inside residual blocks).
 * Status codes are those of tagi_b200.h (TAGI_OK = 0, TAGI_ERR_COMM = 4, ...). One communicator per process.
 */
#ifndef TAGI_B200_COMM_H
#define TAGI_B200_COMM_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

#define TAGI_COMM_ID_BYTES 128

const char *tagi_comm_last_error_string(void);

/* ---- host-only pieces (no GPU, no NCCL needed) ---------------------------------------------------------------- */

/* Rendezvous through a file: rank 0 publishes a blob (written to a temporary name and renamed, so readers never see a
 * partial file); the others fetch it, polling until `timeout_ms` has passed (TAGI_ERR_COMM on expiry: a rank 0 that
 * never joined). Replaces the MPI_Bcast of the ncclUniqueId (src/ddp.cpp:36-40). */
int tagi_rendezvous_publish(const char *path, const void *blob, size_t bytes);
int tagi_rendezvous_fetch(const char *path, void *blob, size_t bytes, int timeout_ms);

/* The same for the communicator id, with a header that tells this job's file from one an earlier job left at the path:
 * publish removes whatever lies at `path` first and records the world size and the time of writing; fetch skips a file
 * with another world size or one written more than timeout_ms before the fetch started, and keeps polling until the
 * deadline (TAGI_ERR_COMM then). `id` is TAGI_COMM_ID_BYTES long. */
int tagi_rendezvous_publish_id(const char *path, const void *id, int world_size);
int tagi_rendezvous_fetch_id(const char *path, void *id, int world_size, int timeout_ms);

/* Bucket plan: tensors i = 0..n-1 of counts[i] floats, in registration order, are packed greedily into buckets of at
 * most bucket_bytes (a tensor larger than the budget gets a bucket of its own); bucket_of[i] receives the bucket
 * index. Returns the number of buckets, or a negative status. */
int tagi_comm_plan_buckets(const size_t *counts, int n, size_t bucket_bytes, int *bucket_of);

/* ---- communicator ---------------------------------------------------------------------------------------------- */

/* Rank 0: create the id (ncclGetUniqueId) into id[TAGI_COMM_ID_BYTES]. */
int tagi_comm_create_id(void *id);
/* All ranks: join. `device` is made current. Replaces NCCLCommunicator's constructor (src/ddp.cpp:27-46). */
int tagi_comm_init(const void *id, int rank, int world_size, int device);
/* Convenience: create the id and tagi_rendezvous_publish_id it (rank 0) or tagi_rendezvous_fetch_id it (others), then
 * join. Rank 0 removes the file again once every rank has joined. */
int tagi_comm_init_file(const char *path, int rank, int world_size, int device, int timeout_ms);
/* Before the communicator is created: upper bound on the CTAs (SMs) one NCCL kernel may use (ncclConfig_t::maxCTAs);
 * 0 = NCCL's default. The exchange runs beside the backward pass's kernels, and every SM NCCL holds is one the
 * tensor-core kernels' tile plan cannot count on (tagi_tc_set_sm_budget). No counterpart in the reference. */
int tagi_comm_set_max_ctas(int max_ctas);
int tagi_comm_rank(void);
int tagi_comm_world_size(void);

/* Register a device tensor of `count` floats for the exchange; call in the order in which backward produces them
 * (last layer first). Returns the tensor's index (>= 0) or a negative status. tagi_comm_finalize_buckets closes the
 * registration and builds the buckets. */
int tagi_comm_register(float *ptr, size_t count);
/* Collective: every rank calls it once, after the same registrations. Tensors of a bucket that lie back to back in device
 * memory (a caller that carves its delta tensors out of one buffer, in registration order) are exchanged as ONE allreduce
 * per run instead of one per tensor, provided every rank found the same runs (checked here with a small allreduce of a
 * hash; any difference and all ranks keep one collective per tensor). */
int tagi_comm_finalize_buckets(size_t bucket_bytes);
int tagi_comm_num_buckets(void);
int tagi_comm_num_tensors(void);     /* tensors registered so far */
int tagi_comm_num_collectives(void); /* allreduce calls one step issues: runs where they were merged, tensors otherwise */
int tagi_comm_bucket_of(int tensor_index);

/* Tell the communicator that tensor `tensor_index` has been written on `compute_stream`. When that completes a
 * bucket, the bucket's allreduce (average != 0: ncclAvg, else ncclSum; src/ddp.cpp:53-57) is launched on the
 * communication stream behind an event recorded on compute_stream. Asynchronous. */
int tagi_comm_tensor_ready(int tensor_index, void *compute_stream, int average);
/* Launch whatever has not been launched yet (tensors never marked ready included). */
int tagi_comm_flush(void *compute_stream, int average);
/* Make compute_stream wait for every launched bucket (stream wait; the host does not block) and re-arm the buckets for
 * the next step. */
int tagi_comm_wait(void *compute_stream);

/* In-place allreduce / broadcast of one buffer on the communication stream, ordered after compute_stream and waited
 * for by compute_stream (replaces Communicator::all_reduce / broadcast, src/ddp.cpp:53-72, for single tensors such as
 * the initial parameter broadcast of sync_base_parameters). */
int tagi_comm_allreduce(float *ptr, size_t count, int average, void *compute_stream);
int tagi_comm_broadcast(float *ptr, size_t count, int root, void *compute_stream);

/* Polls ncclCommGetAsyncError and the CUDA error state (check_cuda_nccl_async, include/cuda_error_checking.cuh:47-74):
 * TAGI_OK or TAGI_ERR_COMM with a message; never exits the process. */
int tagi_comm_check(void);
/* Host waits until everything launched on the communication stream has finished (this rank only). */
int tagi_comm_sync_stream(void);
/* Barrier over the ranks: a one-float allreduce that every rank must enter, then tagi_comm_sync_stream. Replaces
 * Communicator::barrier (src/ddp.cpp:59-62: stream synchronise + MPI_Barrier). */
int tagi_comm_barrier(void);
int tagi_comm_destroy(void);

#ifdef __cplusplus
}
#endif
#endif
