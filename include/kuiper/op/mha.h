// op::MultiHeadAttention (kuiper/include/op/mha.h:6-27, kuiper/source/op/mha.cpp:5-56): inputs
// 0 = query, 1 = score scratch (accepted, never used: scores are not materialised), 2 = key
// cache, 3 = value cache; output 0 = attention output.  With only the reference's setters it
// attends over the reference's contiguous cache.  set_paged(...) switches it to the block
// pool: batched queries, device block table and sequence lengths.
#ifndef KUIPER_INCLUDE_OP_MHA_H_
#define KUIPER_INCLUDE_OP_MHA_H_
#include <cmath>

#include "layer.h"
#include "op/kernels/kernels_interface.h"

namespace op {
// Paged-cache arguments shared by the attention layers (new; no reference counterpart).
struct PagedArgs {
  bool enabled = false;
  tensor::Tensor block_table;  // int32 [batch, max_blocks] on the device
  tensor::Tensor seq_lens;     // int32 [batch] on the device: tokens cached, the new one included
  int32_t batch = 0;
  int64_t num_blocks = 0;      // blocks in the pool (0: ids are not range-checked)
  // Optional: the plan of this decode step (kpx_decode_plan_bytes() bytes on the device, made
  // by MultiHeadAttention::plan_decode_step after the step's lengths were written and before the
  // first layer's attention).  Every layer of the step may carry the same plan.
  tensor::Tensor plan;
};

class MultiHeadAttention : public op::Layer {
 public:
  explicit MultiHeadAttention(base::DeviceType device_type, int32_t layer_index, int32_t kv_mul, int32_t kv_dim,
                              int32_t seq_len, int32_t head_num, int32_t head_size)
      : Layer(device_type, LayerType::kLayerMHA, "MultiHead"), layer_index_(layer_index), kv_mul_(kv_mul),
        kv_dim_(kv_dim), seq_len_(seq_len), head_num_(head_num), head_size_(head_size) {
    reset_input_size(5);
    reset_output_size(1);
  }

  void set_pos(int32_t pos) { pos_ = pos; }
  void set_layer_idx(int32_t layer_idx) { layer_index_ = layer_idx; }
  // Paged mode: inputs 2/3 are the layer's K and V pools [num_blocks][kv_heads][16][head_size].
  void set_paged(const tensor::Tensor& block_table, const tensor::Tensor& seq_lens, int32_t batch,
                 int64_t num_blocks = 0) {
    paged_.enabled = true;
    paged_.block_table = block_table;
    paged_.seq_lens = seq_lens;
    paged_.batch = batch;
    paged_.num_blocks = num_blocks;
  }
  // the plan of the decode step (MultiHeadAttention::plan_decode_step); an empty tensor: none
  void set_plan(const tensor::Tensor& plan) { paged_.plan = plan; }
  const PagedArgs& paged_args() const { return paged_; }

  base::Status check() const override {
    const base::DataType dt = get_input(0).data_type();
    for (int32_t i : {0, 2, 3}) {
      base::Status s = check_tensor(get_input(i), device_type_, dt);
      if (!s) {
        s.set_err_msg("The input tensor " + std::to_string(i) + " error in the mha layer.");
        return s;
      }
    }
    return check_tensor(get_output(0), device_type_, dt);
  }

  base::Status forward() override {
    base::Status st = check();
    if (!st) return st;
    if (device_type_ != base::DeviceType::kDeviceCUDA)
      return base::error::FunctionNotImplement("the KV-cache path is CUDA only");
    if (!paged_.enabled) {
      kernel::get_mha_kernel(device_type_)(pos_, head_num_, layer_index_, seq_len_, kv_dim_, kv_mul_, head_size_,
                                           get_output(0), get_input(0), get_input(1), get_input(2), get_input(3),
                                           device_type_, cuda_config_ ? cuda_config_.get() : nullptr);
      return kernel::detail::taken_status(cuda_config_.get());
    }
    return paged_decode(get_input(0), get_output(0), get_input(2), get_input(3), head_num_, kv_dim_ / head_size_,
                        head_size_, paged_, cuda_config_.get());
  }

  // Batched single-query attention over a block pool (shared by the flash-attention layers).
  static base::Status paged_decode(const tensor::Tensor& query, const tensor::Tensor& out,
                                   const tensor::Tensor& k_pool, const tensor::Tensor& v_pool, int32_t head_num,
                                   int32_t kv_heads, int32_t head_size, const PagedArgs& pa,
                                   kernel::CudaConfig* config) {
    kpx_kv_layout lay;
    int rc = kpx_layout_paged(&lay, kernel::detail::kpx_dtype(k_pool), kv_heads, head_size, 16);
    if (rc != KPX_OK) return base::Status(rc, kpx_status_string(rc));
    lay.num_blocks = pa.num_blocks;
    const float scale = 1.f / std::sqrt(static_cast<float>(head_size));
    if (!pa.plan.is_empty() && config) {
      // with a plan: the workspace form (the plan shortens every launch's prologue)
      const int64_t need = kpx_decode_workspace_bytes(pa.batch, head_num, kv_heads, head_size);
      if (need >= 0 && config->ensure_kv_workspace(static_cast<size_t>(need))) {
        rc = kpx_paged_decode_planned(const_cast<uint8_t*>(out.ptr<uint8_t>()), query.ptr<uint8_t>(),
                                      k_pool.ptr<uint8_t>(), v_pool.ptr<uint8_t>(), &lay,
                                      pa.block_table.ptr<int32_t>(),
                                      pa.block_table.get_dim(pa.block_table.dims_size() - 1),
                                      pa.seq_lens.ptr<int32_t>(), 0, pa.batch, head_num, scale, config->kv_workspace,
                                      static_cast<int64_t>(config->kv_workspace_bytes), pa.plan.ptr<uint8_t>(), 0,
                                      config->stream);
        return rc == KPX_OK ? base::error::Success() : base::Status(rc, kpx_status_string(rc));
      }
    }
    rc = kernel::detail::decode_any(const_cast<uint8_t*>(out.ptr<uint8_t>()), query.ptr<uint8_t>(),
                                    k_pool.ptr<uint8_t>(), v_pool.ptr<uint8_t>(), &lay,
                                    pa.block_table.ptr<int32_t>(),
                                    pa.block_table.get_dim(pa.block_table.dims_size() - 1),
                                    pa.seq_lens.ptr<int32_t>(), 0, pa.batch, head_num, scale, config);
    return rc == KPX_OK ? base::error::Success() : base::Status(rc, kpx_status_string(rc));
  }

  // Once per decode step, after the step's lengths are in pa.seq_lens: fills pa.plan, which the
  // attention layers of all the model's layers then carry (set_paged with the same PagedArgs).
  // `k_pool`: any layer's K pool (for the cache's element type).
  static base::Status plan_decode_step(const PagedArgs& pa, const tensor::Tensor& k_pool, int32_t head_num,
                                       int32_t kv_heads, int32_t head_size, kernel::CudaConfig* config) {
    if (pa.plan.is_empty()) return base::error::InvalidArgument("plan_decode_step: no plan buffer");
    kpx_kv_layout lay;
    int rc = kpx_layout_paged(&lay, kernel::detail::kpx_dtype(k_pool), kv_heads, head_size, 16);
    if (rc != KPX_OK) return base::Status(rc, kpx_status_string(rc));
    lay.num_blocks = pa.num_blocks;
    rc = kpx_decode_plan(const_cast<uint8_t*>(pa.plan.ptr<uint8_t>()), static_cast<int64_t>(pa.plan.byte_size()), &lay,
                         pa.block_table.ptr<int32_t>(), pa.block_table.get_dim(pa.block_table.dims_size() - 1),
                         pa.seq_lens.ptr<int32_t>(), 0, pa.batch, head_num, config ? config->stream : nullptr);
    return rc == KPX_OK ? base::error::Success() : base::Status(rc, kpx_status_string(rc));
  }

 private:
  int32_t layer_index_ = 0;
  int32_t pos_ = 0;
  int32_t kv_mul_ = 0;
  int32_t kv_dim_ = 0;
  int32_t seq_len_ = 0;
  int32_t head_num_ = 0;
  int32_t head_size_ = 0;
  PagedArgs paged_;
};
}  // namespace op
#endif  // KUIPER_INCLUDE_OP_MHA_H_
