// kernel::CudaConfig: the per-model CUDA context the layers share
// (kuiper/include/base/cuda_config.h:17-185).  Of the reference's members only the stream is
// on the KV-cache path; cuBLAS handle, graph context and fp16 GEMM workspaces belong to the
// weight GEMMs.  New: a device scratch for the paged prefill kernels, grown on demand the
// way the reference grows its fp16 workspaces (ensure_fp16_workspace, :109-146).
#ifndef KUIPER_INCLUDE_BASE_CUDA_CONFIG_H_
#define KUIPER_INCLUDE_BASE_CUDA_CONFIG_H_
#include <cuda_runtime_api.h>

#include <cstddef>

#include "kpx.h"

namespace kernel {

struct CudaConfig {
  cudaStream_t stream = nullptr;
  bool use_cuda_graph = false;
  void* kv_workspace = nullptr;  // zero-initialised scratch for kpx_paged_prefill / kpx_paged_decode
  size_t kv_workspace_bytes = 0;
  // The kernel::*_cu free functions return void, as the reference's do; a library status other
  // than KPX_OK that one of them met is kept here (the first since the last take_status()), so
  // that the layer's forward() can hand it to the model instead of going on with stale data.
  int last_status = KPX_OK;

  CudaConfig() = default;
  ~CudaConfig() {
    if (kv_workspace) cudaFree(kv_workspace);
    if (stream) cudaStreamDestroy(stream);
  }
  CudaConfig(const CudaConfig&) = delete;
  CudaConfig& operator=(const CudaConfig&) = delete;

  void init(bool enable_graph = false) {
    if (!stream) cudaStreamCreate(&stream);
    use_cuda_graph = enable_graph;
  }

  void note_status(int rc) {
    if (rc != KPX_OK && last_status == KPX_OK) last_status = rc;
  }
  int take_status() {
    const int rc = last_status;
    last_status = KPX_OK;
    return rc;
  }

  // Make sure the scratch holds `bytes`; (re)allocation synchronises the device, so size it
  // once before the hot loop.  Returns false if the allocation failed.
  bool ensure_kv_workspace(size_t bytes) {
    if (bytes <= kv_workspace_bytes) return true;
    if (kv_workspace) cudaFree(kv_workspace);
    kv_workspace = nullptr;
    kv_workspace_bytes = 0;
    if (cudaMalloc(&kv_workspace, bytes) != cudaSuccess) return false;
    kv_workspace_bytes = bytes;
    return kpx_workspace_init(kv_workspace, static_cast<int64_t>(bytes), stream) == KPX_OK;
  }
};

}  // namespace kernel
#endif  // KUIPER_INCLUDE_BASE_CUDA_CONFIG_H_
