// tensor::Tensor: shape + element type + a shared Buffer, the argument type of every kuiper
// kernel and layer (kuiper/include/tensor/tensor.h:11-105).  Only what the KV-cache path uses
// is here: construction (owning or around an external pointer), ptr<T>() / ptr<T>(index),
// dims, sizes, device type, reshape, to_cuda / to_cpu copies.
#ifndef KUIPER_INCLUDE_TENSOR_TENSOR_H_
#define KUIPER_INCLUDE_TENSOR_TENSOR_H_
#include <cuda_runtime_api.h>

#include <memory>
#include <numeric>
#include <vector>

#include "base/base.h"
#include "base/buffer.h"

namespace tensor {

class Tensor {
 public:
  explicit Tensor() = default;
  explicit Tensor(base::DataType data_type, int32_t dim0, bool need_alloc = false,
                  std::shared_ptr<base::DeviceAllocator> alloc = nullptr, void* ptr = nullptr)
      : Tensor(data_type, std::vector<int32_t>{dim0}, need_alloc, std::move(alloc), ptr) {}
  explicit Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, bool need_alloc = false,
                  std::shared_ptr<base::DeviceAllocator> alloc = nullptr, void* ptr = nullptr)
      : Tensor(data_type, std::vector<int32_t>{dim0, dim1}, need_alloc, std::move(alloc), ptr) {}
  explicit Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2,
                  bool need_alloc = false, std::shared_ptr<base::DeviceAllocator> alloc = nullptr,
                  void* ptr = nullptr)
      : Tensor(data_type, std::vector<int32_t>{dim0, dim1, dim2}, need_alloc, std::move(alloc), ptr) {}
  explicit Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2, int32_t dim3,
                  bool need_alloc = false, std::shared_ptr<base::DeviceAllocator> alloc = nullptr,
                  void* ptr = nullptr)
      : Tensor(data_type, std::vector<int32_t>{dim0, dim1, dim2, dim3}, need_alloc, std::move(alloc), ptr) {}
  explicit Tensor(base::DataType data_type, std::vector<int32_t> dims, bool need_alloc = false,
                  std::shared_ptr<base::DeviceAllocator> alloc = nullptr, void* ptr = nullptr)
      : dims_(std::move(dims)), data_type_(data_type) {
    size_ = 1;
    for (int32_t d : dims_) size_ *= static_cast<size_t>(d);
    if (need_alloc && alloc) {
      allocate(alloc);
    } else if (ptr != nullptr) {
      // wrap memory owned by someone else (never freed here)
      buffer_ = std::make_shared<base::Buffer>(byte_size(), alloc, ptr, true);
    }
  }

  bool is_empty() const { return size_ == 0 || !buffer_ || buffer_->ptr() == nullptr; }
  size_t size() const { return size_; }
  size_t byte_size() const { return size_ * base::DataTypeSize(data_type_); }
  int32_t dims_size() const { return static_cast<int32_t>(dims_.size()); }
  base::DataType data_type() const { return data_type_; }
  int32_t get_dim(int32_t idx) const { return dims_.at(static_cast<size_t>(idx)); }
  const std::vector<int32_t>& dims() const { return dims_; }
  std::shared_ptr<base::Buffer> get_buffer() const { return buffer_; }

  bool allocate(std::shared_ptr<base::DeviceAllocator> allocator, bool need_realloc = false) {
    if (!allocator || byte_size() == 0) return false;
    if (buffer_ && !need_realloc && buffer_->byte_size() >= byte_size()) return true;
    buffer_ = std::make_shared<base::Buffer>(byte_size(), allocator, nullptr);
    return buffer_->ptr() != nullptr;
  }
  bool assign(std::shared_ptr<base::Buffer> buffer) {
    if (!buffer || buffer->byte_size() < byte_size()) return false;
    buffer_ = std::move(buffer);
    return true;
  }
  void reshape(const std::vector<int32_t>& dims) {
    dims_ = dims;
    size_ = 1;
    for (int32_t d : dims_) size_ *= static_cast<size_t>(d);
  }
  void reset(base::DataType data_type, const std::vector<int32_t>& dims) {
    data_type_ = data_type;
    reshape(dims);
    buffer_ = nullptr;
  }

  void set_device_type(base::DeviceType t) const {
    if (buffer_) buffer_->set_device_type(t);
  }
  base::DeviceType device_type() const {
    return buffer_ ? buffer_->device_type() : base::DeviceType::kDeviceUnknown;
  }

  template <typename T>
  T* ptr() { return buffer_ ? reinterpret_cast<T*>(buffer_->ptr()) : nullptr; }
  template <typename T>
  const T* ptr() const { return buffer_ ? reinterpret_cast<const T*>(buffer_->ptr()) : nullptr; }
  template <typename T>
  T* ptr(int64_t index) { return ptr<T>() + index; }
  template <typename T>
  const T* ptr(int64_t index) const { return ptr<T>() + index; }
  template <typename T>
  T& index(int64_t offset) { return *(ptr<T>() + offset); }
  template <typename T>
  const T& index(int64_t offset) const { return *(ptr<T>() + offset); }

  // Moves the data to the device / the host (new owning buffer, synchronous on the stream).
  void to_cuda(cudaStream_t stream = nullptr) { move_to(base::CUDADeviceAllocatorFactory::get_instance(), stream); }
  void to_cpu() { move_to(base::CPUDeviceAllocatorFactory::get_instance(), nullptr); }

  Tensor clone() const {
    Tensor t = *this;
    if (buffer_ && buffer_->allocator()) {
      t.buffer_ = std::make_shared<base::Buffer>(byte_size(), buffer_->allocator(), nullptr);
      copy_bytes(t.buffer_->ptr(), buffer_->ptr(), byte_size(), nullptr);
    }
    return t;
  }

 private:
  static void copy_bytes(void* dst, const void* src, size_t n, cudaStream_t stream) {
    // cudaMemcpyDefault lets the runtime work out the direction from the pointers
    cudaMemcpyAsync(dst, src, n, cudaMemcpyDefault, stream);
    cudaStreamSynchronize(stream);
  }
  void move_to(std::shared_ptr<base::DeviceAllocator> alloc, cudaStream_t stream) {
    if (!buffer_ || buffer_->device_type() == alloc->device_type()) return;
    auto fresh = std::make_shared<base::Buffer>(byte_size(), alloc, nullptr);
    copy_bytes(fresh->ptr(), buffer_->ptr(), byte_size(), stream);
    buffer_ = fresh;
  }

  size_t size_ = 0;
  std::vector<int32_t> dims_;
  std::shared_ptr<base::Buffer> buffer_;
  base::DataType data_type_ = base::DataType::kDataTypeUnknown;
};

}  // namespace tensor
#endif  // KUIPER_INCLUDE_TENSOR_TENSOR_H_
