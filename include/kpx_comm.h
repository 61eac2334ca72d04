/*
 * kpx_comm.h -- C ABI of the one exchange the KV-cache path has between GPUs: the all-gather of
 * per-head attention outputs when a single very long sequence is sharded by KV head (GPU r holds
 * KV heads [r*Hkv/G, (r+1)*Hkv/G) of every block and computes the query heads that read them).
 * Request-parallel operation needs nothing from this file: sequences are independent there.
 *
 * The reference is single-GPU (cudaSetDevice(0) is hard-coded, kuiper/source/model/qwen3.cpp:209;
 * there is no NCCL, MPI or peer copy anywhere in it), so nothing here replaces a reference
 * interface.  The collective is NCCL's all-gather, issued from C++ on the caller's stream into
 * a buffer the caller owns: no allocation, no host synchronisation, and the call can be
 * captured into the same CUDA graph as the attention launch it follows.  One process per GPU.
 * lib/libkpx_comm.so; libkpx.so does not depend on it.
 */
#ifndef KPX_COMM_H_
#define KPX_COMM_H_
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KPX_COMM_API __attribute__((visibility("default")))
#define KPX_COMM_ID_BYTES 128

typedef struct kpx_comm kpx_comm;

/* Rank 0 makes an id and hands its 128 bytes to every rank by its own means (a store, a file,
 * torch.distributed's broadcast of a CPU tensor); every rank then calls kpx_comm_create with it,
 * its CUDA device current.  Status codes are those of kpx.h (0 = ok, 9 = CUDA / NCCL error,
 * 7 = invalid argument). */
KPX_COMM_API int kpx_comm_make_id(void* id_out);
KPX_COMM_API int kpx_comm_create(kpx_comm** out, const void* id, int32_t world, int32_t rank);
/* Destroy every CUDA graph that captured an exchange of this communicator first: NCCL keeps the
 * communicator alive for captured work, and the call would wait for ever. */
KPX_COMM_API int kpx_comm_destroy(kpx_comm* comm);
KPX_COMM_API int kpx_comm_world(const kpx_comm* comm);
KPX_COMM_API int kpx_comm_rank(const kpx_comm* comm);

/* full[r*bytes_per_rank ...] = rank r's `shard` (bytes_per_rank bytes on every rank), for all r,
 * on `stream`.  For one sequence (batch 1) a shard is that rank's heads of the output row,
 * [heads_per_rank * head_size] elements, and `full` is the whole row [num_q_heads * head_size]
 * in head order.  shard may alias full + rank*bytes_per_rank (in place). */
KPX_COMM_API int kpx_allgather_heads(kpx_comm* comm, const void* shard, void* full,
                                     int64_t bytes_per_rank, void* stream);

/* The same for `batch` rows: rank r's shard is [batch, row_bytes_per_rank] and `full` becomes
 * [batch, world*row_bytes_per_rank] (every row in head order): one grouped exchange of
 * batch*world messages, still on `stream`. */
KPX_COMM_API int kpx_allgather_head_rows(kpx_comm* comm, const void* shard, void* full, int32_t batch,
                                         int64_t row_bytes_per_rank, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KPX_COMM_H_ */
