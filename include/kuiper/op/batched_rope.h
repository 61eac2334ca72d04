// op::RoPEGpuPosLayer and op::BatchedRoPELayer (kuiper/include/op/batched_rope.h:20-102,
// kuiper/source/op/batched_rope.cpp): decode RoPE with the position read on the device, and
// RoPE of a prefill chunk whose row s sits at start_pos + s.
#ifndef KUIPER_INCLUDE_OP_BATCHED_ROPE_H_
#define KUIPER_INCLUDE_OP_BATCHED_ROPE_H_
#include "layer.h"
#include "op/kernels/cuda/kv_path_kernels.h"
namespace op {

class RoPEGpuPosLayer : public Layer {
 public:
  explicit RoPEGpuPosLayer(base::DeviceType device_type) : Layer(device_type, LayerType::kLayerRoPe, "RoPEGpuPos") {
    reset_input_size(5);
    reset_output_size(0);
  }
  RoPEGpuPosLayer(base::DeviceType device_type, int32_t dim, int32_t kv_dim, int32_t head_size, bool use_fp16 = false)
      : RoPEGpuPosLayer(device_type) {
    set_dims(dim, kv_dim, head_size);
    use_fp16_ = use_fp16;
  }
  base::Status check() const override {
    if (dim_ <= 0 || kv_dim_ <= 0 || head_size_ <= 0) return base::error::InvalidArgument("Invalid RoPE parameters");
    return base::error::Success();
  }
  // inputs: 0 query, 1 key, 2 position (device int32), 3 sin table, 4 cos table
  base::Status forward() override {
    base::Status st = check();
    if (!st) return st;
    kernel::rope_kernel_cu_gpu_pos(dim_, kv_dim_, head_size_, get_input(0), get_input(1), get_input(2).ptr<int32_t>(),
                                   get_input(3), get_input(4), cuda_config_ ? cuda_config_->stream : nullptr);
    return base::error::Success();
  }
  void set_use_gpu_pos(bool use_gpu_pos) { use_gpu_pos_ = use_gpu_pos; }
  void set_dims(int32_t dim, int32_t kv_dim, int32_t head_size) {
    dim_ = dim;
    kv_dim_ = kv_dim;
    head_size_ = head_size;
  }
  void set_use_fp16(bool use_fp16) { use_fp16_ = use_fp16; }

 private:
  int32_t dim_ = 0, kv_dim_ = 0, head_size_ = 0;
  bool use_fp16_ = false, use_gpu_pos_ = false;
};

class BatchedRoPELayer : public Layer {
 public:
  explicit BatchedRoPELayer(base::DeviceType device_type) : Layer(device_type, LayerType::kLayerRoPe, "BatchedRoPE") {
    reset_input_size(4);
    reset_output_size(0);
  }
  BatchedRoPELayer(base::DeviceType device_type, int32_t dim, int32_t kv_dim, int32_t head_size, int32_t head_num,
                   int32_t kv_head_num)
      : BatchedRoPELayer(device_type) {
    set_dims(dim, kv_dim, head_size, head_num, kv_head_num);
  }
  base::Status check() const override {
    if (dim_ <= 0 || kv_dim_ <= 0 || head_size_ <= 0 || seq_len_ <= 0)
      return base::error::InvalidArgument("Invalid batched RoPE parameters");
    return base::error::Success();
  }
  // inputs: 0 query [n, dim], 1 key [n, kv_dim], 2 sin table, 3 cos table
  base::Status forward() override {
    base::Status st = check();
    if (!st) return st;
    kernel::batched_rope_kernel_cu(start_pos_, seq_len_, dim_, kv_dim_, head_size_, get_input(0), get_input(1),
                                   get_input(2), get_input(3), cuda_config_ ? cuda_config_->stream : nullptr);
    return base::error::Success();
  }
  void set_seq_len(int32_t seq_len) { seq_len_ = seq_len; }
  void set_start_pos(int32_t start_pos) { start_pos_ = start_pos; }
  void set_dims(int32_t dim, int32_t kv_dim, int32_t head_size, int32_t head_num, int32_t kv_head_num) {
    dim_ = dim;
    kv_dim_ = kv_dim;
    head_size_ = head_size;
    head_num_ = head_num;
    kv_head_num_ = kv_head_num;
  }

 private:
  int32_t dim_ = 0, kv_dim_ = 0, head_size_ = 0, head_num_ = 0, kv_head_num_ = 0, seq_len_ = 0, start_pos_ = 0;
};
}  // namespace op
#endif  // KUIPER_INCLUDE_OP_BATCHED_ROPE_H_
