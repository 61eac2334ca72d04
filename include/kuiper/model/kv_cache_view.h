// Views into the KV cache for the layer at hand: where the K and V rows of a token go.
//
// model::slice_kv_cache is the reference's Model::slice_kv_cache
// (kuiper/source/model/model.cpp:348-385) as a free function: the cache is one tensor
// [layers][seq_len][kv_dim] per K and V, the position IS the slot, and the result is a pair of
// kv_dim-long tensors that alias cache[layer][pos] (external-pointer buffers, never freed).
// Offsets are 64-bit here; the reference's int32 arithmetic overflows once
// layers * seq_len * kv_dim passes 2^31.
// model::paged_slot is what takes its place on the block pool: the slot of a position through a
// block table row (slot = block * block_size + position % block_size), which is what
// kpx_append / kpx_rope_append consume.
#ifndef KUIPER_INCLUDE_MODEL_KV_CACHE_VIEW_H_
#define KUIPER_INCLUDE_MODEL_KV_CACHE_VIEW_H_

#include <cstdint>
#include <utility>

#include "base/base.h"
#include "tensor/tensor.h"

namespace model {

inline std::pair<tensor::Tensor, tensor::Tensor> slice_kv_cache(const tensor::Tensor& key_cache,
                                                                const tensor::Tensor& value_cache,
                                                                int32_t layer_idx, int32_t token_pos,
                                                                int32_t seq_len, int32_t kv_dim) {
  const int64_t cache_offset = (int64_t(layer_idx) * seq_len + token_pos) * kv_dim;
  const base::DataType dt = key_cache.data_type();
  const int64_t elt = int64_t(base::DataTypeSize(dt));
  auto* kp = const_cast<uint8_t*>(key_cache.ptr<uint8_t>()) + cache_offset * elt;
  auto* vp = const_cast<uint8_t*>(value_cache.ptr<uint8_t>()) + cache_offset * elt;
  tensor::Tensor key(dt, kv_dim, false, nullptr, kp);
  tensor::Tensor val(dt, kv_dim, false, nullptr, vp);
  key.set_device_type(key_cache.device_type());
  val.set_device_type(value_cache.device_type());
  return {key, val};
}

// Slot of cache position `pos` of a sequence whose block table row is `table_row`
// (host memory); -1 if the position's block is not mapped.
inline int64_t paged_slot(const int32_t* table_row, int32_t max_blocks, int32_t block_size, int32_t pos) {
  if (!table_row || pos < 0 || block_size <= 0 || pos / block_size >= max_blocks) return -1;
  const int32_t block = table_row[pos / block_size];
  return block < 0 ? -1 : int64_t(block) * block_size + pos % block_size;
}

}  // namespace model
#endif  // KUIPER_INCLUDE_MODEL_KV_CACHE_VIEW_H_
