// NCCL-backed exchange of the KV-head-sharded mode (include/kpx_comm.h): communicator set-up and
// the all-gather of per-head attention outputs, issued from C++ on the caller's stream.
#include "kpx_comm.h"

#include <cuda_runtime_api.h>
#include <nccl.h>

#include <cstring>
#include <new>

#include "kpx.h"

static_assert(KPX_COMM_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "id size must match ncclUniqueId");

struct kpx_comm {
  ncclComm_t comm = nullptr;
  int world = 0, rank = 0;
};

namespace {
inline int nccl_status(ncclResult_t r) { return r == ncclSuccess ? KPX_OK : KPX_ERR_CUDA; }
}  // namespace

extern "C" int kpx_comm_make_id(void* id_out) {
  if (!id_out) return KPX_ERR_INVALID_ARGUMENT;
  ncclUniqueId id;
  if (ncclGetUniqueId(&id) != ncclSuccess) return KPX_ERR_CUDA;
  std::memcpy(id_out, &id, sizeof(id));
  return KPX_OK;
}

extern "C" int kpx_comm_create(kpx_comm** out, const void* id, int32_t world, int32_t rank) {
  if (!out || !id || world < 1 || rank < 0 || rank >= world) return KPX_ERR_INVALID_ARGUMENT;
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof(uid));
  kpx_comm* c = new (std::nothrow) kpx_comm;
  if (!c) return KPX_ERR_INTERNAL;
  c->world = world;
  c->rank = rank;
  if (ncclCommInitRank(&c->comm, world, uid, rank) != ncclSuccess) {
    delete c;
    return KPX_ERR_CUDA;
  }
  *out = c;
  return KPX_OK;
}

extern "C" int kpx_comm_destroy(kpx_comm* comm) {
  if (!comm) return KPX_OK;
  ncclResult_t r = comm->comm ? ncclCommDestroy(comm->comm) : ncclSuccess;
  delete comm;
  return nccl_status(r);
}

extern "C" int kpx_comm_world(const kpx_comm* comm) { return comm ? comm->world : 0; }
extern "C" int kpx_comm_rank(const kpx_comm* comm) { return comm ? comm->rank : -1; }

extern "C" int kpx_allgather_heads(kpx_comm* comm, const void* shard, void* full, int64_t bytes_per_rank,
                                   void* stream) {
  if (!comm || !shard || !full || bytes_per_rank <= 0) return KPX_ERR_INVALID_ARGUMENT;
  return nccl_status(ncclAllGather(shard, full, static_cast<size_t>(bytes_per_rank), ncclInt8, comm->comm,
                                   static_cast<cudaStream_t>(stream)));
}

extern "C" int kpx_allgather_head_rows(kpx_comm* comm, const void* shard, void* full, int32_t batch,
                                       int64_t row_bytes_per_rank, void* stream) {
  if (!comm || !shard || !full || batch < 1 || row_bytes_per_rank <= 0) return KPX_ERR_INVALID_ARGUMENT;
  if (batch == 1) return kpx_allgather_heads(comm, shard, full, row_bytes_per_rank, stream);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t full_row = row_bytes_per_rank * comm->world;
  const char* src = static_cast<const char*>(shard);
  char* dst = static_cast<char*>(full);
  // row b of this rank goes to columns [rank*row_bytes, +row_bytes) of row b on every rank
  ncclResult_t r = ncclGroupStart();
  for (int32_t b = 0; b < batch && r == ncclSuccess; ++b) {
    for (int peer = 0; peer < comm->world && r == ncclSuccess; ++peer) {
      r = ncclSend(src + b * row_bytes_per_rank, static_cast<size_t>(row_bytes_per_rank), ncclInt8, peer, comm->comm, s);
      if (r == ncclSuccess)
        r = ncclRecv(dst + b * full_row + peer * row_bytes_per_rank, static_cast<size_t>(row_bytes_per_rank),
                     ncclInt8, peer, comm->comm, s);
    }
  }
  ncclResult_t e = ncclGroupEnd();
  return nccl_status(r != ncclSuccess ? r : e);
}
