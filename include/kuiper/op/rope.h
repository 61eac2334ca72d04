// op::RoPELayer (kuiper/include/op/rope.h:5-19, kuiper/source/op/rope.cpp:7-45): inputs
// 0 = query, 1 = key (rotated in place), 2 = position (int32, device memory here), 3 = sin
// table, 4 = cos table.
#ifndef KUIPER_INCLUDE_OP_ROPE_H_
#define KUIPER_INCLUDE_OP_ROPE_H_
#include "layer.h"
#include "op/kernels/kernels_interface.h"
namespace op {
class RoPELayer : public Layer {
 public:
  explicit RoPELayer(base::DeviceType device_type, int32_t dim, int32_t kv_dim, int32_t head_size)
      : Layer(device_type, LayerType::kLayerRoPe, "RoPe"), dim_(dim), kv_dim_(kv_dim), head_size_(head_size) {
    reset_input_size(5);
    reset_output_size(1);
  }
  base::Status check() const override {
    for (int i = 0; i < 5; ++i)
      if (get_input(i).is_empty()) return base::error::InvalidArgument("The input tensor " + std::to_string(i) + " error in the rope layer.");
    return base::error::Success();
  }
  base::Status forward() override {
    base::Status st = check();
    if (!st) return st;
    kernel::get_rope_kernel(device_type_)(dim_, kv_dim_, head_size_, get_input(0), get_input(1), get_input(2),
                                          get_input(3), get_input(4), cuda_config_ ? cuda_config_->stream : nullptr);
    return base::error::Success();
  }

 private:
  int32_t dim_ = 0, kv_dim_ = 0, head_size_ = 0;
};
}  // namespace op
#endif  // KUIPER_INCLUDE_OP_ROPE_H_
