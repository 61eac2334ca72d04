// op::BaseLayer / op::Layer: input/output slots, device type, CUDA config, the forward(...)
// overloads that fill the slots and run forward() (kuiper/include/op/layer.h:25-155,
// kuiper/source/op/layer.cpp:329-377).  LayerParam (weights) is not on the KV-cache path.
#ifndef KUIPER_INCLUDE_OP_LAYER_H_
#define KUIPER_INCLUDE_OP_LAYER_H_
#include <memory>
#include <string>
#include <vector>

#include "base/base.h"
#include "base/cuda_config.h"
#include "tensor/tensor.h"

namespace op {
enum class LayerType : uint8_t {
  kLayerUnknown = 0, kLayerLinear = 1, kLayerEncode = 2, kLayerEmbedding = 3, kLayerRMSNorm = 4,
  kLayerMatmul = 5, kLayerRoPe = 6, kLayerMHA = 7, kLayerSoftmax = 8, kLayerAdd = 9, kLayerSwiGLU = 10,
};

class BaseLayer {
 public:
  explicit BaseLayer(base::DeviceType device_type, LayerType layer_type, base::DataType data_type,
                     std::string layer_name = "")
      : layer_name_(std::move(layer_name)), layer_type_(layer_type), data_type_(data_type),
        device_type_(device_type) {}
  virtual ~BaseLayer() = default;
  base::DataType data_type() const { return data_type_; }
  LayerType layer_type() const { return layer_type_; }
  virtual base::Status init() = 0;
  virtual base::Status forward() = 0;
  virtual void set_input(int32_t idx, const tensor::Tensor& input) = 0;
  virtual void set_output(int32_t idx, const tensor::Tensor& output) = 0;
  virtual size_t input_size() const = 0;
  virtual size_t output_size() const = 0;
  virtual base::Status check() const = 0;
  virtual tensor::Tensor& get_input(int32_t idx) = 0;
  virtual tensor::Tensor& get_output(int32_t idx) = 0;
  virtual const tensor::Tensor& get_input(int32_t idx) const = 0;
  virtual const tensor::Tensor& get_output(int32_t idx) const = 0;
  const std::string& get_layer_name() const { return layer_name_; }
  void set_layer_name(const std::string& n) { layer_name_ = n; }
  base::DeviceType device_type() const { return device_type_; }
  void set_device_type(base::DeviceType t) { device_type_ = t; }

 protected:
  std::string layer_name_;
  LayerType layer_type_ = LayerType::kLayerUnknown;
  base::DataType data_type_ = base::DataType::kDataTypeUnknown;
  base::DeviceType device_type_ = base::DeviceType::kDeviceUnknown;
};

class Layer : public BaseLayer {
 public:
  explicit Layer(base::DeviceType device_type, LayerType layer_type, std::string layer_name = "")
      : BaseLayer(device_type, layer_type, base::DataType::kDataTypeFp32, std::move(layer_name)) {}

  base::Status init() override { return base::error::Success(); }
  base::Status check() const override { return base::error::FunctionNotImplement("The check function is not implement yet"); }
  base::Status forward() override { return base::error::FunctionNotImplement(""); }

  base::Status check_tensor(const tensor::Tensor& t, base::DeviceType device_type,
                            base::DataType data_type) const {
    if (t.is_empty()) return base::error::InvalidArgument("The tensor parameter is empty.");
    if (t.device_type() != device_type) return base::error::InvalidArgument("The tensor has a wrong device type.");
    if (t.data_type() != data_type) return base::error::InvalidArgument("The tensor has a wrong data type.");
    return base::error::Success();
  }

  base::Status forward(const tensor::Tensor& i1, const tensor::Tensor& o1) {
    set_input(0, i1);
    set_output(0, o1);
    return this->forward();
  }
  base::Status forward(const tensor::Tensor& i1, const tensor::Tensor& i2, const tensor::Tensor& o1) {
    set_input(0, i1);
    set_input(1, i2);
    set_output(0, o1);
    return this->forward();
  }
  base::Status forward(const tensor::Tensor& i1, const tensor::Tensor& i2, const tensor::Tensor& i3,
                       const tensor::Tensor& o1) {
    set_input(0, i1);
    set_input(1, i2);
    set_input(2, i3);
    set_output(0, o1);
    return this->forward();
  }
  base::Status forward(const tensor::Tensor& i1, const tensor::Tensor& i2, const tensor::Tensor& i3,
                       const tensor::Tensor& i4, const tensor::Tensor& o1) {
    set_input(0, i1);
    set_input(1, i2);
    set_input(2, i3);
    set_input(3, i4);
    set_output(0, o1);
    return this->forward();
  }
  base::Status forward(const tensor::Tensor& i1, const tensor::Tensor& i2, const tensor::Tensor& i3,
                       const tensor::Tensor& i4, const tensor::Tensor& i5, const tensor::Tensor& o1) {
    set_input(0, i1);
    set_input(1, i2);
    set_input(2, i3);
    set_input(3, i4);
    set_input(4, i5);
    set_output(0, o1);
    return this->forward();
  }

  void set_input(int32_t idx, const tensor::Tensor& input) override { inputs_.at(static_cast<size_t>(idx)) = input; }
  void set_output(int32_t idx, const tensor::Tensor& output) override { outputs_.at(static_cast<size_t>(idx)) = output; }
  const tensor::Tensor& get_input(int32_t idx) const override { return inputs_.at(static_cast<size_t>(idx)); }
  const tensor::Tensor& get_output(int32_t idx) const override { return outputs_.at(static_cast<size_t>(idx)); }
  tensor::Tensor& get_input(int32_t idx) override { return inputs_.at(static_cast<size_t>(idx)); }
  tensor::Tensor& get_output(int32_t idx) override { return outputs_.at(static_cast<size_t>(idx)); }
  size_t input_size() const override { return inputs_.size(); }
  size_t output_size() const override { return outputs_.size(); }
  void reset_input_size(size_t size) { inputs_.resize(size); }
  void reset_output_size(size_t size) { outputs_.resize(size); }
  virtual void to_cuda() {
    for (auto& t : inputs_) if (!t.is_empty()) t.to_cuda(cuda_config_ ? cuda_config_->stream : nullptr);
    for (auto& t : outputs_) if (!t.is_empty()) t.to_cuda(cuda_config_ ? cuda_config_->stream : nullptr);
  }
  void set_cuda_config(std::shared_ptr<kernel::CudaConfig> config) {
    if (config) cuda_config_ = std::move(config);
  }
  std::shared_ptr<kernel::CudaConfig> cuda_config() const { return cuda_config_; }

 protected:
  std::vector<tensor::Tensor> inputs_;
  std::vector<tensor::Tensor> outputs_;
  std::shared_ptr<kernel::CudaConfig> cuda_config_;
};
}  // namespace op
#endif  // KUIPER_INCLUDE_OP_LAYER_H_
