// The attention / KV-cache helper layers of kuiper/include/op/misc_layers.h that sit on the
// KV-cache path: MHAGpuPosLayer (:27-40), BatchedMHALayer (:45-60), FusedKVCacheUpdateLayer
// (:134-147), CopyToKVCacheLayer (:167-178), FlashAttentionDecodeGpuPosLayer (:183-205), and
// SinCosCacheLayer (:10-22) because the RoPE'd K it feeds must be reproducible.  The other
// classes of that header (matmul helper, M-RoPE, per-dim RMSNorm) are not on the path.
// Each has the reference's constructor and direct forward(...) overload; forward() without
// arguments is "not implemented" exactly as in the reference (misc_layers.cpp).
#ifndef KUIPER_INCLUDE_OP_MISC_LAYERS_H_
#define KUIPER_INCLUDE_OP_MISC_LAYERS_H_
#include "layer.h"
#include "op/kernels/cuda/kv_path_kernels.h"

namespace op {

#define KUIPER_B200_MISC_LAYER_HEAD(cls, name)                                                   \
 public:                                                                                         \
  explicit cls(base::DeviceType device_type) : Layer(device_type, LayerType::kLayerUnknown, name) {} \
  base::Status check() const override { return base::error::Success(); }                         \
  base::Status forward() override {                                                              \
    return base::error::FunctionNotImplement(name " requires direct forward with parameters");   \
  }

class SinCosCacheLayer : public Layer {
  KUIPER_B200_MISC_LAYER_HEAD(SinCosCacheLayer, "SinCosCache")
  base::Status forward(int32_t head_size, int32_t seq_len, const tensor::Tensor& sin_cache,
                       const tensor::Tensor& cos_cache, float theta = 1000000.0f) {
    kernel::sin_cos_cache_calc_cu(head_size, seq_len, sin_cache, cos_cache,
                                  cuda_config_ ? cuda_config_->stream : nullptr, theta);
    return base::error::Success();
  }
};

class MHAGpuPosLayer : public Layer {
  KUIPER_B200_MISC_LAYER_HEAD(MHAGpuPosLayer, "MHAGpuPos")
  base::Status forward(const int32_t* pos_ptr, int32_t head_num, int32_t layer_idx, int32_t seq_len, int32_t kv_dim,
                       int32_t kv_mul, int32_t head_size, tensor::Tensor& mha_output, const tensor::Tensor& query,
                       tensor::Tensor& score_storage, const tensor::Tensor& key_cache,
                       const tensor::Tensor& val_cache) {
    kernel::mha_kernel_cu_gpu_pos(pos_ptr, head_num, layer_idx, seq_len, kv_dim, kv_mul, head_size, mha_output, query,
                                  score_storage, key_cache, val_cache, device_type_, cuda_config_.get());
    return kernel::detail::taken_status(cuda_config_.get());
  }
};

class BatchedMHALayer : public Layer {
  KUIPER_B200_MISC_LAYER_HEAD(BatchedMHALayer, "BatchedMHA")
  base::Status forward(int32_t start_pos, int32_t seq_len, int32_t head_num, int32_t layer_idx, int32_t max_seq_len,
                       int32_t dim, int32_t kv_dim, int32_t kv_mul, int32_t head_size, tensor::Tensor& mha_output,
                       const tensor::Tensor& query, tensor::Tensor& score_storage, const tensor::Tensor& key_cache,
                       const tensor::Tensor& val_cache) {
    if (!cuda_config_) return base::error::InvalidArgument("prefill needs a CudaConfig (it owns the scratch)");
    kernel::batched_mha_kernel_cu(start_pos, seq_len, head_num, layer_idx, max_seq_len, dim, kv_dim, kv_mul,
                                  head_size, mha_output, query, score_storage, key_cache, val_cache, device_type_,
                                  cuda_config_.get());
    return kernel::detail::taken_status(cuda_config_.get());
  }
};

class FusedKVCacheUpdateLayer : public Layer {
  KUIPER_B200_MISC_LAYER_HEAD(FusedKVCacheUpdateLayer, "FusedKVCacheUpdate")
  base::Status forward(const tensor::Tensor& key, const tensor::Tensor& value, const tensor::Tensor& key_cache,
                       const tensor::Tensor& val_cache, int32_t layer_idx, int32_t start_pos, int32_t seq_len,
                       int32_t kv_dim, int32_t max_seq_len) {
    kernel::fused_kv_cache_update_cu(key, value, const_cast<tensor::Tensor&>(key_cache),
                                     const_cast<tensor::Tensor&>(val_cache), layer_idx, start_pos, seq_len, kv_dim,
                                     max_seq_len, cuda_config_ ? cuda_config_->stream : nullptr);
    return base::error::Success();
  }
};

class CopyToKVCacheLayer : public Layer {
  KUIPER_B200_MISC_LAYER_HEAD(CopyToKVCacheLayer, "CopyToKVCache")
  base::Status forward(const tensor::Tensor& kv_cache, const tensor::Tensor& kv_data, const int32_t* pos_gpu,
                       int32_t kv_dim, int32_t layer_idx, int32_t seq_len) {
    cudaStream_t stream = cuda_config_ ? cuda_config_->stream : nullptr;
    if (base::DataTypeSize(kv_cache.data_type()) == 2)
      kernel::copy_to_kv_cache_kernel_fp16(const_cast<uint8_t*>(kv_cache.ptr<uint8_t>()), kv_data.ptr<uint8_t>(),
                                           pos_gpu, kv_dim, layer_idx, seq_len, stream);
    else
      kernel::copy_to_kv_cache_kernel(const_cast<float*>(kv_cache.ptr<float>()), kv_data.ptr<float>(), pos_gpu,
                                      kv_dim, layer_idx, seq_len, stream);
    return base::error::Success();
  }
};

class FlashAttentionDecodeGpuPosLayer : public Layer {
  KUIPER_B200_MISC_LAYER_HEAD(FlashAttentionDecodeGpuPosLayer, "FlashAttentionDecodeGpuPos")
  void set_attention_type(base::AttentionType type) { attention_type_ = type; }
  base::AttentionType get_attention_type() const { return attention_type_; }
  base::Status forward(const int32_t* pos_gpu, int32_t head_num, int32_t kv_head_num, int32_t head_size,
                       int32_t kv_mul, int32_t layer_idx, int32_t seq_len, int32_t kv_dim,
                       const tensor::Tensor& query, const tensor::Tensor& mha_output,
                       const tensor::Tensor& key_cache, const tensor::Tensor& val_cache) {
    kernel::flash_attention_decode_fp16_gpu_pos_cu(pos_gpu, head_num, kv_head_num, head_size, kv_mul, layer_idx,
                                                   seq_len, kv_dim, query, mha_output, key_cache, val_cache,
                                                   cuda_config_.get());
    return kernel::detail::taken_status(cuda_config_.get());
  }

 private:
  base::AttentionType attention_type_ = base::AttentionType::kAttentionFlash1;
};

#undef KUIPER_B200_MISC_LAYER_HEAD
}  // namespace op
#endif  // KUIPER_INCLUDE_OP_MISC_LAYERS_H_
