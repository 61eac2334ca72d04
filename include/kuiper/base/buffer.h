// base::DeviceAllocator / base::Buffer: the minimum of kuiper/include/base/alloc.h:20-115 and
// buffer.h:8-50 that the KV-cache path's argument type (tensor::Tensor) needs.  A Buffer
// either owns memory obtained from an allocator or wraps an external pointer that it never
// frees (the reference's use_external flag), which is how cache rows are aliased.
#ifndef KUIPER_INCLUDE_BASE_BUFFER_H_
#define KUIPER_INCLUDE_BASE_BUFFER_H_
#include <cuda_runtime_api.h>

#include <cstdlib>
#include <cstring>
#include <memory>

#include "base.h"

namespace base {

class DeviceAllocator {
 public:
  explicit DeviceAllocator(DeviceType t) : device_type_(t) {}
  virtual ~DeviceAllocator() = default;
  virtual DeviceType device_type() const { return device_type_; }
  virtual void* allocate(size_t byte_size) const = 0;
  virtual void release(void* ptr) const = 0;

 private:
  DeviceType device_type_;
};

class CPUDeviceAllocator : public DeviceAllocator {
 public:
  CPUDeviceAllocator() : DeviceAllocator(DeviceType::kDeviceCPU) {}
  void* allocate(size_t n) const override { return n ? std::malloc(n) : nullptr; }
  void release(void* p) const override { std::free(p); }
};

class CUDADeviceAllocator : public DeviceAllocator {
 public:
  CUDADeviceAllocator() : DeviceAllocator(DeviceType::kDeviceCUDA) {}
  void* allocate(size_t n) const override {
    void* p = nullptr;
    if (n == 0 || cudaMalloc(&p, n) != cudaSuccess) return nullptr;
    return p;
  }
  void release(void* p) const override {
    if (p) cudaFree(p);
  }
};

struct CPUDeviceAllocatorFactory {
  static std::shared_ptr<CPUDeviceAllocator> get_instance() {
    static std::shared_ptr<CPUDeviceAllocator> inst = std::make_shared<CPUDeviceAllocator>();
    return inst;
  }
};
struct CUDADeviceAllocatorFactory {
  static std::shared_ptr<CUDADeviceAllocator> get_instance() {
    static std::shared_ptr<CUDADeviceAllocator> inst = std::make_shared<CUDADeviceAllocator>();
    return inst;
  }
};

class Buffer : public NoCopyable, public std::enable_shared_from_this<Buffer> {
 public:
  Buffer() = default;
  Buffer(size_t byte_size, std::shared_ptr<DeviceAllocator> allocator = nullptr, void* ptr = nullptr,
         bool use_external = false)
      : byte_size_(byte_size), ptr_(ptr), use_external_(use_external), allocator_(std::move(allocator)) {
    if (!ptr_ && allocator_) {
      device_type_ = allocator_->device_type();
      use_external_ = false;
      ptr_ = allocator_->allocate(byte_size_);
    } else if (allocator_) {
      device_type_ = allocator_->device_type();
    }
  }
  ~Buffer() {
    if (!use_external_ && ptr_ && allocator_) allocator_->release(ptr_);
  }
  bool allocate() {
    if (!allocator_ || byte_size_ == 0) return false;
    use_external_ = false;
    ptr_ = allocator_->allocate(byte_size_);
    return ptr_ != nullptr;
  }
  void* ptr() { return ptr_; }
  const void* ptr() const { return ptr_; }
  size_t byte_size() const { return byte_size_; }
  std::shared_ptr<DeviceAllocator> allocator() const { return allocator_; }
  DeviceType device_type() const { return device_type_; }
  void set_device_type(DeviceType t) { device_type_ = t; }
  bool is_external() const { return use_external_; }

 private:
  size_t byte_size_ = 0;
  void* ptr_ = nullptr;
  bool use_external_ = false;
  DeviceType device_type_ = DeviceType::kDeviceUnknown;
  std::shared_ptr<DeviceAllocator> allocator_;
};

}  // namespace base
#endif  // KUIPER_INCLUDE_BASE_BUFFER_H_
