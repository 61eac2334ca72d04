// Kernel registry of the KV-cache path: the function-pointer types and get_*_kernel()
// selectors of kuiper/source/op/kernels/kernels_interface.h:22-73 for the entries on the path
// (MHA, RoPE).  kDeviceCUDA returns the sm_100a implementation.  This library has no CPU
// kernels: asking for kDeviceCPU ends like the reference's switch does for an unknown device
// (a fatal message), not with a silent fallback.
#ifndef KUIPER_OP_KERNELS_INTERFACE_H_
#define KUIPER_OP_KERNELS_INTERFACE_H_
#include "base/cuda_config.h"
#include "op/kernels/cuda/kv_path_kernels.h"
#include "tensor/tensor.h"

namespace kernel {
typedef void (*MHAKernel)(int32_t pos, int32_t head_num, int32_t layer_index, int32_t seq_len, int32_t kv_dim,
                          int32_t kv_mul, int32_t head_size, const tensor::Tensor& mha_out,
                          const tensor::Tensor& query_tensor, const tensor::Tensor& score_tensor,
                          const tensor::Tensor& key_cache_tensor, const tensor::Tensor& value_cache_tensor,
                          base::DeviceType device_type, CudaConfig*);

typedef void (*RoPEKernel)(int32_t dim, int32_t kv_dim, int32_t head_size, const tensor::Tensor& input_q,
                           const tensor::Tensor& input_k, const tensor::Tensor& input_pos,
                           const tensor::Tensor& sin_cache, const tensor::Tensor& cos_cache, void* stream);

inline MHAKernel get_mha_kernel(base::DeviceType device_type) {
  if (device_type == base::DeviceType::kDeviceCUDA) return mha_kernel_cu;
  std::fprintf(stderr, "Unknown device type for get an mha kernel (this library is CUDA only).\n");
  std::abort();
}

inline RoPEKernel get_rope_kernel(base::DeviceType device_type) {
  if (device_type == base::DeviceType::kDeviceCUDA) return rope_kernel_cu;
  std::fprintf(stderr, "Unknown device type for get a rope kernel (this library is CUDA only).\n");
  std::abort();
}
}  // namespace kernel
#endif  // KUIPER_OP_KERNELS_INTERFACE_H_
