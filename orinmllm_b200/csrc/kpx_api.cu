// Entry points that are not kernels: status strings, layouts, device info,
// workspace status word.
#include <mutex>

#include "kpx_common.cuh"

namespace kpx {

const DeviceInfo& device_info() {
  static DeviceInfo infos[64];
  static std::mutex mu;
  static DeviceInfo none;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return none;
  }
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo& di = infos[dev];
  if (!di.ok) {
    int sm = 0, smem = 0;
    if (cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess) {
      di.sm_count = sm;
      di.smem_optin = smem;
      di.ok = true;
    } else {
      (void)cudaGetLastError();
    }
  }
  return di;
}

}  // namespace kpx

using namespace kpx;

extern "C" const char* kpx_status_string(int status) {
  switch (status) {
    case KPX_OK: return "ok";
    case KPX_ERR_UNIMPLEMENTED: return "not implemented for these dimensions or types";
    case KPX_ERR_INTERNAL: return "internal error";
    case KPX_ERR_INVALID_ARGUMENT: return "invalid argument";
    case KPX_ERR_OUT_OF_BLOCKS: return "block pool exhausted";
    case KPX_ERR_CUDA: return "CUDA runtime error or no CUDA device";
    case KPX_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case KPX_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case KPX_ERR_REFCOUNT: return "block reference count would become negative";
    case KPX_ERR_NOT_FOUND: return "not found";
    case KPX_ERR_STATIC_SCRATCH_LIMIT:
      return "beyond the limits of the built-in scratch array (num_kv_heads * head groups > 16)";
    default: return "unknown status";
  }
}

extern "C" int kpx_abi_version(void) { return 1; }

extern "C" int kpx_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

static int fill_layout(kpx_kv_layout* out, int32_t dtype, int32_t kvh, int32_t hs, int32_t bs) {
  if (!out || kvh <= 0 || hs <= 0 || bs <= 0) return KPX_ERR_INVALID_ARGUMENT;
  if (dtype != KPX_F16 && dtype != KPX_BF16 && dtype != KPX_F32) return KPX_ERR_INVALID_ARGUMENT;
  out->dtype = dtype;
  out->num_kv_heads = kvh;
  out->head_size = hs;
  out->block_size = bs;
  out->num_blocks = 0;
  return KPX_OK;
}

extern "C" int kpx_layout_paged(kpx_kv_layout* out, int32_t dtype, int32_t num_kv_heads,
                                int32_t head_size, int32_t block_size) {
  int rc = fill_layout(out, dtype, num_kv_heads, head_size, block_size);
  if (rc != KPX_OK) return rc;
  out->token_stride = head_size;
  out->head_stride = int64_t(block_size) * head_size;
  out->block_stride = int64_t(num_kv_heads) * block_size * head_size;
  return KPX_OK;
}

extern "C" int kpx_layout_contiguous(kpx_kv_layout* out, int32_t dtype, int32_t num_kv_heads,
                                     int32_t head_size, int32_t block_size) {
  int rc = fill_layout(out, dtype, num_kv_heads, head_size, block_size);
  if (rc != KPX_OK) return rc;
  int64_t kv_dim = int64_t(num_kv_heads) * head_size;
  out->token_stride = kv_dim;
  out->head_stride = head_size;
  out->block_stride = int64_t(block_size) * kv_dim;
  return KPX_OK;
}

namespace {
// Header of a workspace: word 0 = sticky status (the kernels raise it), word 1 = a mark that
// kpx_workspace_init has been here, bytes 8..15 = the size it was given, so that the workspace
// can be wiped again without asking (and is not, if the header is not ours).
constexpr int32_t kWorkspaceMark = 0x4b505857;  // "KPXW"
__global__ void workspace_note_size(int64_t* header, int64_t bytes) {
  reinterpret_cast<int32_t*>(header)[1] = kWorkspaceMark;
  header[1] = bytes;
}

int wipe_workspace(void* workspace, int64_t workspace_bytes, cudaStream_t s) {
  KPX_CUDA_TRY(cudaMemsetAsync(workspace, 0, size_t(workspace_bytes), s));
  workspace_note_size<<<1, 1, 0, s>>>(static_cast<int64_t*>(workspace), workspace_bytes);
  KPX_CUDA_TRY(cudaGetLastError());
  return KPX_OK;
}
}  // namespace

extern "C" int kpx_workspace_init(void* workspace, int64_t workspace_bytes, void* stream) {
  if (!workspace || workspace_bytes < 256 || (reinterpret_cast<uintptr_t>(workspace) & 15))
    return KPX_ERR_INVALID_ARGUMENT;
  return wipe_workspace(workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int kpx_workspace_status(void* workspace, void* stream) {
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15)) return KPX_ERR_INVALID_ARGUMENT;
  int64_t header[2] = {0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KPX_CUDA_TRY(cudaMemcpyAsync(header, workspace, sizeof(header), cudaMemcpyDeviceToHost, s));
  KPX_CUDA_TRY(cudaStreamSynchronize(s));
  const int32_t st = static_cast<int32_t>(header[0] & 0xffffffff);
  const bool ours = static_cast<int32_t>(header[0] >> 32) == kWorkspaceMark;
  if (st == KPX_ERR_DEVICE_TIMEOUT && ours && header[1] >= 256) {
    // warps that gave up never counted their pieces: the counters in the workspace are stale and
    // the next launch would assemble at the wrong count, so the whole workspace starts over
    int rc = wipe_workspace(workspace, header[1], s);
    if (rc != KPX_OK) return rc;
  } else if (st != 0) {
    KPX_CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(int32_t), s));
  }
  return st;
}
