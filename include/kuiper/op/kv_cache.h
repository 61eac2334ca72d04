// op::KVCacheLayer (kuiper/include/op/kv_cache.h:19-41, kuiper/source/op/kv_cache.cpp:8-61):
// inputs 0 = the new K (or V) row(s), 1 = the cache, 2 = position tensor in device memory.
// With only the reference's setters: cache[layer][*pos][:] <- input, one token.  Paged mode
// (new): set_slot_mapping(slots, n) scatters n rows into the block pool in input 1.
#ifndef KUIPER_INCLUDE_OP_KV_CACHE_H_
#define KUIPER_INCLUDE_OP_KV_CACHE_H_
#include "layer.h"
#include "op/kernels/cuda/kv_path_kernels.h"

namespace op {
class KVCacheLayer : public Layer {
 public:
  explicit KVCacheLayer(base::DeviceType device_type) : Layer(device_type, LayerType::kLayerUnknown, "KVCache") {
    reset_input_size(3);
    reset_output_size(0);
  }
  KVCacheLayer(base::DeviceType device_type, int32_t kv_dim, int32_t seq_len, bool use_fp16 = false)
      : KVCacheLayer(device_type) {
    kv_dim_ = kv_dim;
    seq_len_ = seq_len;
    use_fp16_ = use_fp16;
  }

  base::Status check() const override {
    if (kv_dim_ <= 0 || (seq_len_ <= 0 && !paged_)) return base::error::InvalidArgument("Invalid KV cache parameters");
    return base::error::Success();
  }

  base::Status forward() override {
    base::Status st = check();
    if (!st) return st;
    const tensor::Tensor& input = get_input(0);
    const tensor::Tensor& cache = get_input(1);
    cudaStream_t stream = cuda_config_ ? cuda_config_->stream : nullptr;
    if (paged_) {
      kpx_kv_layout lay;
      kpx_layout_paged(&lay, kernel::detail::kpx_dtype(cache), kv_dim_ / head_size_, head_size_, 16);
      lay.num_blocks = num_blocks_;
      int rc = kpx_append(const_cast<uint8_t*>(cache.ptr<uint8_t>()), nullptr, &lay, input.ptr<uint8_t>(), nullptr,
                          slots_.ptr<int64_t>(), nullptr, 0, num_tokens_, stream);
      return rc == KPX_OK ? base::error::Success() : base::Status(rc, kpx_status_string(rc));
    }
    const int32_t* pos = get_input(2).ptr<int32_t>();
    if (use_fp16_ || base::DataTypeSize(cache.data_type()) == 2) {
      kernel::copy_to_kv_cache_kernel_fp16(const_cast<uint8_t*>(cache.ptr<uint8_t>()), input.ptr<uint8_t>(), pos,
                                           kv_dim_, layer_index_, seq_len_, stream);
    } else {
      kernel::copy_to_kv_cache_kernel(const_cast<float*>(cache.ptr<float>()), input.ptr<float>(), pos, kv_dim_,
                                      layer_index_, seq_len_, stream);
    }
    return base::error::Success();
  }

  void set_layer_index(int32_t layer_index) { layer_index_ = layer_index; }
  void set_use_gpu_pos(bool use_gpu_pos) { use_gpu_pos_ = use_gpu_pos; }
  void set_dims(int32_t kv_dim, int32_t seq_len) {
    kv_dim_ = kv_dim;
    seq_len_ = seq_len;
  }
  void set_use_fp16(bool use_fp16) { use_fp16_ = use_fp16; }
  // Paged mode: input 1 is one layer's K (or V) pool; slots is an int64 device tensor [num_tokens].
  void set_slot_mapping(const tensor::Tensor& slots, int32_t num_tokens, int32_t head_size = 128,
                        int64_t num_blocks = 0) {
    paged_ = true;
    slots_ = slots;
    num_tokens_ = num_tokens;
    head_size_ = head_size;
    num_blocks_ = num_blocks;
  }

 private:
  int32_t kv_dim_ = 0, seq_len_ = 0, layer_index_ = 0;
  bool use_fp16_ = false, use_gpu_pos_ = false;
  bool paged_ = false;
  tensor::Tensor slots_;
  int32_t num_tokens_ = 0, head_size_ = 128;
  int64_t num_blocks_ = 0;
};
}  // namespace op
#endif  // KUIPER_INCLUDE_OP_KV_CACHE_H_
