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

extern "C" int kpx_workspace_init(void* workspace, int64_t workspace_bytes, void* stream) {
  if (!workspace || workspace_bytes < 256) return KPX_ERR_INVALID_ARGUMENT;
  KPX_CUDA_TRY(cudaMemsetAsync(workspace, 0, size_t(workspace_bytes), static_cast<cudaStream_t>(stream)));
  return KPX_OK;
}

extern "C" int kpx_workspace_status(void* workspace, void* stream) {
  if (!workspace) return KPX_ERR_INVALID_ARGUMENT;
  int32_t st = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KPX_CUDA_TRY(cudaMemcpyAsync(&st, workspace, sizeof(st), cudaMemcpyDeviceToHost, s));
  KPX_CUDA_TRY(cudaStreamSynchronize(s));
  if (st != 0) KPX_CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(st), s));
  return st;
}
