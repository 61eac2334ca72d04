// C entry points over the reference project's own CPU kernels, for the checker.
//
// TEST INFRASTRUCTURE.  This file is compiled together with the UNMODIFIED reference
// sources (taken from the reference checkout where it lies, never copied):
//   kuiper/source/op/kernels/cpu/{mha,matmul,softmax,scale_sum,rope,rmsnorm}_kernel.cpp
//   kuiper/source/tensor/tensor.cpp, kuiper/source/base/{base,buffer,alloc,alloc_cpu,alloc_cu}.cpp
// against the stand-in headers under shim/ (glog, Armadillo).  It adds only what those
// files need from the rest of the reference and cannot be had without its CUDA sources:
// the three registry look-ups mha_kernel calls (kernels_interface.h:51-73), returning the
// reference's CPU functions; and plain-C wrappers that put raw pointers into
// tensor::Tensor views the way mha_kernel.cpp:24-27 does.
#include <cstdint>
#include <memory>

#include "base/alloc.h"
#include "base/base.h"
#include "tensor/tensor.h"

// declarations as in kuiper/source/op/kernels/cpu/*.h
#include "../cpu/matmul_kernel.h"
#include "../cpu/mha_kernel.h"
#include "../cpu/rmsnorm_kernel.h"
#include "../cpu/rope_kernel.h"
#include "../cpu/scale_sum_kernel.h"
#include "../cpu/softmax_kernel.h"
#include "../kernels_interface.h"

namespace kernel {
// kernels_interfaces.cpp:43-52,94-101 and the scale-sum entry: CPU branch only (the CUDA
// branch needs the reference's .cu files, which are what this repository replaces).
MatmulKernel get_matmul_kernel(base::DeviceType device_type) {
  CHECK(device_type == base::DeviceType::kDeviceCPU) << "checker build: CPU kernels only";
  return matmul_kernel_cpu;
}
SoftmaxInplaceKernel get_softmax_kernel(base::DeviceType device_type) {
  CHECK(device_type == base::DeviceType::kDeviceCPU) << "checker build: CPU kernels only";
  return static_cast<SoftmaxInplaceKernel>(softmax_inplace_cpu);
}
ScaleSumKernel get_scale_sum_kernel(base::DeviceType device_type) {
  CHECK(device_type == base::DeviceType::kDeviceCPU) << "checker build: CPU kernels only";
  return scale_sum_kernel_cpu;
}
}  // namespace kernel

namespace {
tensor::Tensor view(base::DataType dt, std::vector<int32_t> dims, const void* ptr) {
  tensor::Tensor t(dt, std::move(dims), false, nullptr, const_cast<void*>(ptr));
  t.set_device_type(base::DeviceType::kDeviceCPU);
  return t;
}
}  // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

// kernel::mha_kernel (cpu/mha_kernel.cpp:5-61) with the MHAKernel argument list.
REF_API void ref_mha(int32_t pos, int32_t head_num, int32_t layer_index, int32_t seq_len,
                     int32_t kv_dim, int32_t kv_mul, int32_t head_size, int32_t layer_num,
                     float* mha_out, const float* query, float* score, const float* key_cache,
                     const float* value_cache) {
  using base::DataType;
  tensor::Tensor out = view(DataType::kDataTypeFp32, {head_num * head_size}, mha_out);
  tensor::Tensor q = view(DataType::kDataTypeFp32, {head_num * head_size}, query);
  tensor::Tensor sc = view(DataType::kDataTypeFp32, {head_num, seq_len}, score);
  tensor::Tensor kc = view(DataType::kDataTypeFp32, {layer_num, seq_len, kv_dim}, key_cache);
  tensor::Tensor vc = view(DataType::kDataTypeFp32, {layer_num, seq_len, kv_dim}, value_cache);
  kernel::mha_kernel(pos, head_num, layer_index, seq_len, kv_dim, kv_mul, head_size, out, q, sc, kc,
                     vc, base::DeviceType::kDeviceCPU, nullptr);
}

// kernel::sin_cos_cache_calc_cpu (cpu/rope_kernel.cpp:44-56, the Qwen branch: theta 1e6).
REF_API void ref_sin_cos_cache(int32_t head_size, int32_t max_seq_len, float* sin_cache,
                               float* cos_cache) {
  kernel::sin_cos_cache_calc_cpu(head_size, max_seq_len, sin_cache, cos_cache);
}

// kernel::rope_kernel_cpu (cpu/rope_kernel.cpp:58-82), q [dim] and k [kv_dim] in place.
REF_API void ref_rope(int32_t dim, int32_t kv_dim, int32_t head_size, float* q, float* k,
                      int32_t pos, int32_t max_seq_len, const float* sin_cache,
                      const float* cos_cache) {
  using base::DataType;
  tensor::Tensor tq = view(DataType::kDataTypeFp32, {dim}, q);
  tensor::Tensor tk = view(DataType::kDataTypeFp32, {kv_dim}, k);
  int32_t pos_host = pos;
  tensor::Tensor tp = view(DataType::kDataTypeInt32, {1}, &pos_host);
  tensor::Tensor ts = view(DataType::kDataTypeFp32, {max_seq_len, head_size}, sin_cache);
  tensor::Tensor tc = view(DataType::kDataTypeFp32, {max_seq_len, head_size}, cos_cache);
  kernel::rope_kernel_cpu(dim, kv_dim, head_size, tq, tk, tp, ts, tc, nullptr);
}

// kernel::rmsnorm_kernel_cpu (cpu/rmsnorm_kernel.cpp:4-34) on one row of `dim` values.
REF_API void ref_rmsnorm(int32_t dim, const float* input, const float* weight, float* output) {
  using base::DataType;
  tensor::Tensor ti = view(DataType::kDataTypeFp32, {dim}, input);
  tensor::Tensor tw = view(DataType::kDataTypeFp32, {dim}, weight);
  tensor::Tensor to = view(DataType::kDataTypeFp32, {dim}, output);
  kernel::rmsnorm_kernel_cpu(ti, tw, to, nullptr);
}

// kernel::softmax_inplace_cpu (cpu/softmax_kernel.cpp:4-15).
REF_API void ref_softmax(float* x, int32_t size) {
  tensor::Tensor t = view(base::DataType::kDataTypeFp32, {size}, x);
  kernel::softmax_inplace_cpu(t, nullptr);
}

// 1 when the stand-in reductions run in plain index order (-DSHIM_ARMA_SEQUENTIAL).
REF_API int ref_sequential_reductions(void) {
#ifdef SHIM_ARMA_SEQUENTIAL
  return 1;
#else
  return 0;
#endif
}
