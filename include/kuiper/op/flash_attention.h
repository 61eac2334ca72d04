// op::FlashAttentionDecodeLayer / op::FlashAttentionPrefillLayer with the constructors,
// setters, input slots and direct forward(...) overloads of kuiper/include/op/flash_attention.h
// :19-115 (implementation kuiper/source/op/flash_attention.cpp:11-226).  The AttentionType
// (MHA / Flash1 / Flash2) is kept as a property: all three are served by the same kernels.
// Paged mode (new): set_paged(...) on the decode layer, set_paged_prefill(...) on the prefill
// layer; inputs 2/3 are then the layer's K/V block pools.
#ifndef KUIPER_INCLUDE_OP_FLASH_ATTENTION_H_
#define KUIPER_INCLUDE_OP_FLASH_ATTENTION_H_
#include <vector>

#include "layer.h"
#include "mha.h"

namespace op {

class FlashAttentionDecodeLayer : public Layer {
 public:
  explicit FlashAttentionDecodeLayer(base::DeviceType device_type)
      : Layer(device_type, LayerType::kLayerMHA, "FlashAttentionDecode") {
    reset_input_size(5);
    reset_output_size(1);
  }
  FlashAttentionDecodeLayer(base::DeviceType device_type, int32_t head_num, int32_t kv_head_num, int32_t head_size,
                            int32_t kv_mul, int32_t seq_len, int32_t kv_dim, bool use_fp16 = false)
      : FlashAttentionDecodeLayer(device_type) {
    set_dims(head_num, kv_head_num, head_size, kv_mul, seq_len, kv_dim);
    use_fp16_ = use_fp16;
  }

  base::Status check() const override {
    if (head_num_ <= 0 || kv_head_num_ <= 0 || head_size_ <= 0 || kv_dim_ <= 0)
      return base::error::InvalidArgument("Invalid flash attention decode parameters");
    if (get_input(0).is_empty() || get_input(1).is_empty() || get_input(2).is_empty() || get_input(3).is_empty())
      return base::error::InvalidArgument("flash attention decode: an input tensor is empty");
    if (use_gpu_pos_ && !paged_.enabled && get_input(4).is_empty())
      return base::error::InvalidArgument("flash attention decode: use_gpu_pos needs the position tensor");
    return base::error::Success();
  }

  // inputs: 0 query, 1 output (written in place), 2 key cache, 3 value cache, 4 device position
  base::Status forward() override {
    base::Status st = check();
    if (!st) return st;
    if (paged_.enabled)
      return MultiHeadAttention::paged_decode(get_input(0), get_input(1), get_input(2), get_input(3), head_num_,
                                              kv_head_num_, head_size_, paged_, cuda_config_.get());
    if (use_gpu_pos_) {
      kernel::flash_attention_decode_fp16_gpu_pos_cu(get_input(4).ptr<int32_t>(), head_num_, kv_head_num_, head_size_,
                                                     kv_mul_, layer_index_, seq_len_, kv_dim_, get_input(0),
                                                     get_input(1), get_input(2), get_input(3), cuda_config_.get());
      return kernel::detail::taken_status(cuda_config_.get());
    }
    return forward(pos_, head_num_, kv_head_num_, head_size_, kv_mul_, layer_index_, seq_len_, kv_dim_,
                   get_input(0), get_input(1), get_input(2), get_input(3));
  }

  base::Status forward(int32_t pos, int32_t head_num, int32_t kv_head_num, int32_t head_size, int32_t kv_mul,
                       int32_t layer_idx, int32_t seq_len, int32_t kv_dim, const tensor::Tensor& query,
                       const tensor::Tensor& mha_output, const tensor::Tensor& key_cache,
                       const tensor::Tensor& val_cache) {
    kernel::flash_attention_decode_cu(pos, head_num, kv_head_num, head_size, kv_mul, layer_idx, seq_len, kv_dim,
                                      query, mha_output, key_cache, val_cache, cuda_config_.get());
    return kernel::detail::taken_status(cuda_config_.get());
  }

  void set_layer_index(int32_t layer_index) { layer_index_ = layer_index; }
  void set_pos(int32_t pos) { pos_ = pos; }
  void set_use_gpu_pos(bool use_gpu_pos) { use_gpu_pos_ = use_gpu_pos; }
  void set_dims(int32_t head_num, int32_t kv_head_num, int32_t head_size, int32_t kv_mul, int32_t seq_len,
                int32_t kv_dim) {
    head_num_ = head_num;
    kv_head_num_ = kv_head_num;
    head_size_ = head_size;
    kv_mul_ = kv_mul;
    seq_len_ = seq_len;
    kv_dim_ = kv_dim;
  }
  void set_use_fp16(bool use_fp16) { use_fp16_ = use_fp16; }
  void set_attention_type(base::AttentionType type) { attention_type_ = type; }
  base::AttentionType get_attention_type() const { return attention_type_; }
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

 private:
  int32_t head_num_ = 0, kv_head_num_ = 0, head_size_ = 0, kv_mul_ = 0, seq_len_ = 0, kv_dim_ = 0;
  int32_t layer_index_ = 0, pos_ = 0;
  bool use_fp16_ = false, use_gpu_pos_ = false;
  base::AttentionType attention_type_ = base::AttentionType::kAttentionFlash1;
  PagedArgs paged_;
};

class FlashAttentionPrefillLayer : public Layer {
 public:
  explicit FlashAttentionPrefillLayer(base::DeviceType device_type)
      : Layer(device_type, LayerType::kLayerMHA, "FlashAttentionPrefill") {
    reset_input_size(4);
    reset_output_size(1);
  }
  FlashAttentionPrefillLayer(base::DeviceType device_type, int32_t head_num, int32_t kv_head_num, int32_t head_size,
                             int32_t seq_len, bool use_fp16 = false)
      : FlashAttentionPrefillLayer(device_type) {
    set_dims(head_num, kv_head_num, head_size, seq_len);
    use_fp16_ = use_fp16;
  }

  base::Status check() const override {
    if (head_num_ <= 0 || kv_head_num_ <= 0 || head_size_ <= 0)
      return base::error::InvalidArgument("Invalid flash attention prefill parameters");
    for (int i = 0; i < 4; ++i)
      if (get_input(i).is_empty()) return base::error::InvalidArgument("flash attention prefill: empty input tensor");
    return base::error::Success();
  }

  // inputs: 0 query [n, dim], 1 output [n, dim], 2 key cache, 3 value cache
  base::Status forward() override {
    base::Status st = check();
    if (!st) return st;
    if (paged_.enabled) return paged_forward();
    return forward(start_pos_, cur_seq_len_, head_num_, kv_head_num_, head_size_, head_num_ / kv_head_num_,
                   layer_idx_, max_seq_len_, kv_head_num_ * head_size_, get_input(0), get_input(1), get_input(2),
                   get_input(3));
  }

  base::Status forward(int32_t start_pos, int32_t seq_len, int32_t head_num, int32_t kv_head_num, int32_t head_size,
                       int32_t kv_mul, int32_t layer_idx, int32_t max_seq_len, int32_t kv_dim,
                       const tensor::Tensor& query, const tensor::Tensor& output, const tensor::Tensor& key_cache,
                       const tensor::Tensor& val_cache) {
    if (!cuda_config_) return base::error::InvalidArgument("prefill needs a CudaConfig (it owns the scratch)");
    kernel::flash_attention_prefill_cu(start_pos, seq_len, head_num, kv_head_num, head_size, kv_mul, layer_idx,
                                       max_seq_len, kv_dim, query, output, key_cache, val_cache, cuda_config_.get());
    return kernel::detail::taken_status(cuda_config_.get());
  }

  void set_cur_seq_len(int32_t seq_len) { cur_seq_len_ = seq_len; }
  void set_start_pos(int32_t start_pos) { start_pos_ = start_pos; }
  void set_layer_index(int32_t layer_idx) { layer_idx_ = layer_idx; }
  void set_dims(int32_t head_num, int32_t kv_head_num, int32_t head_size, int32_t max_seq_len) {
    head_num_ = head_num;
    kv_head_num_ = kv_head_num;
    head_size_ = head_size;
    max_seq_len_ = max_seq_len;
  }
  void set_use_fp16(bool use_fp16) { use_fp16_ = use_fp16; }
  void set_attention_type(base::AttentionType type) { attention_type_ = type; }
  base::AttentionType get_attention_type() const { return attention_type_; }
  // Paged chunked prefill of several sequences at once: query rows [cu_q_lens[b], cu_q_lens[b+1])
  // belong to sequence b (row b of the block table) and start at position start_pos[b].
  void set_paged_prefill(const tensor::Tensor& block_table, const std::vector<int32_t>& cu_q_lens,
                         const std::vector<int32_t>& start_pos, int64_t num_blocks = 0) {
    paged_.enabled = true;
    paged_.block_table = block_table;
    paged_.batch = static_cast<int32_t>(start_pos.size());
    paged_.num_blocks = num_blocks;
    cu_q_lens_ = cu_q_lens;
    starts_ = start_pos;
  }

 private:
  base::Status paged_forward() {
    if (!cuda_config_) return base::error::InvalidArgument("prefill needs a CudaConfig (it owns the scratch)");
    const int32_t total_q = cu_q_lens_.empty() ? 0 : cu_q_lens_.back();
    const int64_t need = kpx_prefill_workspace_bytes(total_q, head_num_, kv_head_num_, head_size_);
    if (need < 0 || !cuda_config_->ensure_kv_workspace(static_cast<size_t>(need)))
      return base::error::InternalError("prefill scratch allocation failed");
    kpx_kv_layout lay;
    kpx_layout_paged(&lay, kernel::detail::kpx_dtype(get_input(2)), kv_head_num_, head_size_, 16);
    lay.num_blocks = paged_.num_blocks;
    const tensor::Tensor& bt = paged_.block_table;
    int rc = kpx_paged_prefill(const_cast<uint8_t*>(get_input(1).ptr<uint8_t>()), get_input(0).ptr<uint8_t>(),
                               get_input(2).ptr<uint8_t>(), get_input(3).ptr<uint8_t>(), &lay, bt.ptr<int32_t>(),
                               bt.get_dim(bt.dims_size() - 1), cu_q_lens_.data(), starts_.data(), paged_.batch,
                               head_num_, 1.f / std::sqrt(static_cast<float>(head_size_)),
                               cuda_config_->kv_workspace, static_cast<int64_t>(cuda_config_->kv_workspace_bytes),
                               cuda_config_->stream);
    return rc == KPX_OK ? base::error::Success() : base::Status(rc, kpx_status_string(rc));
  }

  int32_t head_num_ = 0, kv_head_num_ = 0, head_size_ = 0, max_seq_len_ = 0;
  int32_t cur_seq_len_ = 0, start_pos_ = 0, layer_idx_ = 0;
  bool use_fp16_ = false;
  base::AttentionType attention_type_ = base::AttentionType::kAttentionFlash1;
  PagedArgs paged_;
  std::vector<int32_t> cu_q_lens_, starts_;
};

}  // namespace op
#endif  // KUIPER_INCLUDE_OP_FLASH_ATTENTION_H_
