// kernel::*_cu free functions of the KV-cache path with the reference's names and argument
// lists, each a few lines that unwrap the Tensors and call the C ABI (include/kpx.h).  They
// keep the reference's contiguous-cache semantics: cache [layer][seq_len][kv_dim], position
// either a host int or a device int32.  Like the reference they return void; a non-zero
// status from the library is reported on stderr (the reference does not check its launches).
//
// Declarations replaced (reference paths):
//   cuda/mha_kernel.cuh:4-26, cuda/flash_attention_kernel.cuh:27-234,
//   cuda/kv_cache_kernel.cuh:24-33, cuda/fused_kernels.cuh:53-64, cuda/rope_kernel.cuh:5-28.
#ifndef KUIPER_OP_KERNELS_CUDA_KV_PATH_KERNELS_H_
#define KUIPER_OP_KERNELS_CUDA_KV_PATH_KERNELS_H_
#include <cmath>
#include <cstdio>

#include "base/cuda_config.h"
#include "kpx.h"
#include "tensor/tensor.h"

namespace kernel {
namespace detail {
inline void report(int rc, const char* what, CudaConfig* config = nullptr) {
  if (rc == KPX_OK) return;
  std::fprintf(stderr, "[kuiper-b200] %s: %s\n", what, kpx_status_string(rc));
  if (config) config->note_status(rc);
}
// What the void functions below met since the last look (kept in the CudaConfig), as a Status
// for the layer's forward() to return.
inline base::Status taken_status(CudaConfig* config) {
  const int rc = config ? config->take_status() : KPX_OK;
  return rc == KPX_OK ? base::error::Success() : base::Status(rc, kpx_status_string(rc));
}
// Single-query attention through the library.  First choice is the entry point with built-in
// scratch (nothing to allocate, nothing to pass); a head layout beyond its limit (for example
// 32 KV heads, plain multi-head attention) falls back to kpx_paged_decode with the config's
// workspace, grown once.  Without a config there is nowhere to keep a workspace and the limit
// is returned.
inline int decode_any(void* out, const void* q, const void* k, const void* v, const kpx_kv_layout* lay,
                      const int32_t* table, int32_t max_blocks, const int32_t* seq_lens, int32_t len_bias,
                      int32_t batch, int32_t head_num, float scale, CudaConfig* config) {
  void* stream = config ? config->stream : nullptr;
  int rc = kpx_paged_decode_static(out, q, k, v, lay, table, max_blocks, seq_lens, len_bias, batch, head_num,
                                   scale, stream);
  if (rc != KPX_ERR_STATIC_SCRATCH_LIMIT || !config) return rc;
  const int64_t need = kpx_decode_workspace_bytes(batch, head_num, lay->num_kv_heads, lay->head_size);
  if (need < 0 || !config->ensure_kv_workspace(static_cast<size_t>(need))) return KPX_ERR_WORKSPACE_TOO_SMALL;
  return kpx_paged_decode(out, q, k, v, lay, table, max_blocks, seq_lens, len_bias, batch, head_num, scale,
                          config->kv_workspace, static_cast<int64_t>(config->kv_workspace_bytes), stream);
}
inline int32_t kpx_dtype(const tensor::Tensor& t) {
  switch (t.data_type()) {
    case base::DataType::kDataTypeFp16: return KPX_F16;
    case base::DataType::kDataTypeBf16: return KPX_BF16;
    default: return KPX_F32;
  }
}
inline void* stream_of(const CudaConfig* config) { return config ? config->stream : nullptr; }
inline kpx_kv_layout contiguous_layout(int32_t dtype, int32_t kv_dim, int32_t head_size) {
  kpx_kv_layout lay;
  kpx_layout_contiguous(&lay, dtype, kv_dim / head_size, head_size, 16);
  return lay;
}
// byte pointer of layer `layer_index` of a cache tensor [layers][seq_len][kv_dim]
inline uint8_t* layer_base(const tensor::Tensor& cache, int32_t layer_index, int32_t seq_len, int32_t kv_dim) {
  const int64_t elems = int64_t(layer_index) * seq_len * kv_dim;
  return const_cast<uint8_t*>(cache.ptr<uint8_t>()) + elems * int64_t(base::DataTypeSize(cache.data_type()));
}
// single-query attention over rows 0..len-1 of the layer's cache
inline void decode_contiguous(const int32_t* pos_dev, int32_t host_len, int32_t head_num, int32_t layer_index,
                              int32_t seq_len, int32_t kv_dim, int32_t head_size, const tensor::Tensor& out,
                              const tensor::Tensor& query, const tensor::Tensor& key_cache,
                              const tensor::Tensor& value_cache, CudaConfig* config, const char* what) {
  kpx_kv_layout lay = contiguous_layout(kpx_dtype(key_cache), kv_dim, head_size);
  lay.num_blocks = (seq_len + lay.block_size - 1) / lay.block_size;  // rows the layer's cache holds
  report(decode_any(const_cast<uint8_t*>(out.ptr<uint8_t>()), query.ptr<uint8_t>(),
                    layer_base(key_cache, layer_index, seq_len, kv_dim),
                    layer_base(value_cache, layer_index, seq_len, kv_dim), &lay, nullptr, 0, pos_dev,
                    pos_dev ? 1 : host_len, 1, head_num, 1.f / std::sqrt(static_cast<float>(head_size)), config),
         what, config);
}
// causal attention of seq_len query rows at start_pos.. over the layer's cache
inline void prefill_contiguous(int32_t start_pos, int32_t n, int32_t head_num, int32_t layer_index,
                               int32_t max_seq_len, int32_t kv_dim, int32_t head_size,
                               const tensor::Tensor& out, const tensor::Tensor& query,
                               const tensor::Tensor& key_cache, const tensor::Tensor& value_cache,
                               CudaConfig* config, const char* what) {
  if (!config) {
    report(KPX_ERR_INVALID_ARGUMENT, "prefill needs a CudaConfig (it owns the scratch)");
    return;
  }
  kpx_kv_layout lay = contiguous_layout(kpx_dtype(key_cache), kv_dim, head_size);
  const int64_t need = kpx_prefill_workspace_bytes(n, head_num, kv_dim / head_size, head_size);
  if (need < 0 || !config->ensure_kv_workspace(static_cast<size_t>(need))) {
    report(KPX_ERR_WORKSPACE_TOO_SMALL, what, config);
    return;
  }
  const int32_t cu[2] = {0, n};
  report(kpx_paged_prefill(const_cast<uint8_t*>(out.ptr<uint8_t>()), query.ptr<uint8_t>(),
                           layer_base(key_cache, layer_index, max_seq_len, kv_dim),
                           layer_base(value_cache, layer_index, max_seq_len, kv_dim), &lay, nullptr, 0, cu,
                           &start_pos, 1, head_num, 1.f / std::sqrt(static_cast<float>(head_size)),
                           config->kv_workspace, static_cast<int64_t>(config->kv_workspace_bytes),
                           config->stream), what, config);
}
}  // namespace detail

// ---- MHA (fp32 in the reference; any cache dtype here) ------------------------------------
inline void mha_kernel_cu(int32_t pos, int32_t head_num, int32_t layer_index, int32_t seq_len, int32_t kv_dim,
                          int32_t kv_mul, int32_t head_size, const tensor::Tensor& mha_out,
                          const tensor::Tensor& query_tensor, const tensor::Tensor& score_tensor,
                          const tensor::Tensor& key_cache_tensor, const tensor::Tensor& value_cache_tensor,
                          base::DeviceType device_type, CudaConfig* config) {
  UNUSED(kv_mul); UNUSED(score_tensor); UNUSED(device_type);  // scores are never materialised
  detail::decode_contiguous(nullptr, pos + 1, head_num, layer_index, seq_len, kv_dim, head_size, mha_out,
                            query_tensor, key_cache_tensor, value_cache_tensor, config,
                            "mha_kernel_cu");
}
inline void mha_kernel_cu_gpu_pos(const int32_t* pos_ptr, int32_t head_num, int32_t layer_index, int32_t seq_len,
                                  int32_t kv_dim, int32_t kv_mul, int32_t head_size,
                                  const tensor::Tensor& mha_out, const tensor::Tensor& query_tensor,
                                  const tensor::Tensor& score_tensor, const tensor::Tensor& key_cache_tensor,
                                  const tensor::Tensor& value_cache_tensor, base::DeviceType device_type,
                                  CudaConfig* config) {
  UNUSED(kv_mul); UNUSED(score_tensor); UNUSED(device_type);
  detail::decode_contiguous(pos_ptr, 0, head_num, layer_index, seq_len, kv_dim, head_size, mha_out, query_tensor,
                            key_cache_tensor, value_cache_tensor, config,
                            "mha_kernel_cu_gpu_pos");
}
inline void batched_mha_kernel_cu(int32_t start_pos, int32_t seq_len, int32_t head_num, int32_t layer_index,
                                  int32_t max_seq_len, int32_t dim, int32_t kv_dim, int32_t kv_mul,
                                  int32_t head_size, const tensor::Tensor& mha_out,
                                  const tensor::Tensor& query_tensor, const tensor::Tensor& score_tensor,
                                  const tensor::Tensor& key_cache_tensor, const tensor::Tensor& value_cache_tensor,
                                  base::DeviceType device_type, CudaConfig* config) {
  UNUSED(dim); UNUSED(kv_mul); UNUSED(score_tensor); UNUSED(device_type);
  detail::prefill_contiguous(start_pos, seq_len, head_num, layer_index, max_seq_len, kv_dim, head_size, mha_out,
                             query_tensor, key_cache_tensor, value_cache_tensor, config, "batched_mha_kernel_cu");
}

// ---- flash attention: all reference variants (FA1 / FA2, fp32 / fp16, host / device pos)
// ---- are the same two operations here ----------------------------------------------------
#define KUIPER_B200_DECODE_CU(name)                                                                        \
  inline void name(int32_t pos, int32_t head_num, int32_t kv_head_num, int32_t head_size, int32_t kv_mul, \
                   int32_t layer_index, int32_t max_seq_len, int32_t kv_dim, const tensor::Tensor& query, \
                   const tensor::Tensor& output, const tensor::Tensor& key_cache,                         \
                   const tensor::Tensor& value_cache, CudaConfig* config) {                               \
    UNUSED(kv_head_num); UNUSED(kv_mul);                                                                   \
    detail::decode_contiguous(nullptr, pos + 1, head_num, layer_index, max_seq_len, kv_dim, head_size,    \
                              output, query, key_cache, value_cache, config, #name);                      \
  }
#define KUIPER_B200_DECODE_GPU_POS_CU(name)                                                                \
  inline void name(const int32_t* pos_ptr, int32_t head_num, int32_t kv_head_num, int32_t head_size,      \
                   int32_t kv_mul, int32_t layer_index, int32_t max_seq_len, int32_t kv_dim,              \
                   const tensor::Tensor& query, const tensor::Tensor& output,                             \
                   const tensor::Tensor& key_cache, const tensor::Tensor& value_cache,                    \
                   CudaConfig* config) {                                                                   \
    UNUSED(kv_head_num); UNUSED(kv_mul);                                                                   \
    detail::decode_contiguous(pos_ptr, 0, head_num, layer_index, max_seq_len, kv_dim, head_size, output,  \
                              query, key_cache, value_cache, config, #name);                              \
  }
#define KUIPER_B200_PREFILL_CU(name)                                                                       \
  inline void name(int32_t start_pos, int32_t seq_len, int32_t head_num, int32_t kv_head_num,             \
                   int32_t head_size, int32_t kv_mul, int32_t layer_index, int32_t max_seq_len,           \
                   int32_t kv_dim, const tensor::Tensor& query, const tensor::Tensor& output,             \
                   const tensor::Tensor& key_cache, const tensor::Tensor& value_cache,                    \
                   CudaConfig* config) {                                                                   \
    UNUSED(kv_head_num); UNUSED(kv_mul);                                                                   \
    detail::prefill_contiguous(start_pos, seq_len, head_num, layer_index, max_seq_len, kv_dim, head_size, \
                               output, query, key_cache, value_cache, config, #name);                     \
  }
KUIPER_B200_DECODE_CU(flash_attention_decode_cu)
KUIPER_B200_DECODE_CU(flash_attention_decode_fp16_cu)
KUIPER_B200_DECODE_CU(flash_attention2_decode_cu)
KUIPER_B200_DECODE_CU(flash_attention2_decode_fp16_cu)
KUIPER_B200_DECODE_GPU_POS_CU(flash_attention_decode_fp16_gpu_pos_cu)
KUIPER_B200_DECODE_GPU_POS_CU(flash_attention2_decode_fp16_gpu_pos_cu)
KUIPER_B200_PREFILL_CU(flash_attention_prefill_cu)
KUIPER_B200_PREFILL_CU(flash_attention_prefill_fp16_cu)
KUIPER_B200_PREFILL_CU(flash_attention2_prefill_cu)
KUIPER_B200_PREFILL_CU(flash_attention2_prefill_fp16_cu)
#undef KUIPER_B200_DECODE_CU
#undef KUIPER_B200_DECODE_GPU_POS_CU
#undef KUIPER_B200_PREFILL_CU

// ---- KV append ---------------------------------------------------------------------------
namespace detail {
inline void append_row(void* cache, const void* src, const int32_t* pos, int32_t kv_dim, int32_t layer_idx,
                       int32_t seq_len, int32_t dtype, cudaStream_t stream, const char* what) {
  // head_size only shapes the 16-byte vector walk; any divisor of kv_dim with 16-byte rows works
  const int32_t hs = kv_dim % 128 == 0 ? 128 : kv_dim;
  kpx_kv_layout lay = contiguous_layout(dtype, kv_dim, hs);
  uint8_t* base = static_cast<uint8_t*>(cache) + int64_t(layer_idx) * seq_len * kv_dim * (dtype == KPX_F32 ? 4 : 2);
  report(kpx_append(base, nullptr, &lay, src, nullptr, nullptr, pos, 0, 1, stream), what);
}
}  // namespace detail
inline void copy_to_kv_cache_kernel(float* kv_cache, const float* src, const int32_t* pos, int32_t kv_dim,
                                    int32_t layer_idx, int32_t seq_len, cudaStream_t stream) {
  detail::append_row(kv_cache, src, pos, kv_dim, layer_idx, seq_len, KPX_F32, stream, "copy_to_kv_cache_kernel");
}
// `half` in the reference signature; any 16-bit element type is moved bit for bit
inline void copy_to_kv_cache_kernel_fp16(void* kv_cache, const void* src, const int32_t* pos, int32_t kv_dim,
                                         int32_t layer_idx, int32_t seq_len, cudaStream_t stream) {
  detail::append_row(kv_cache, src, pos, kv_dim, layer_idx, seq_len, KPX_F16, stream, "copy_to_kv_cache_kernel_fp16");
}
inline void fused_kv_cache_update_cu(const tensor::Tensor& key_out, const tensor::Tensor& value_out,
                                     tensor::Tensor& key_cache, tensor::Tensor& value_cache, int layer_idx,
                                     int start_pos, int seq_len, int kv_dim, int max_seq_len, cudaStream_t stream) {
  const int32_t hs = kv_dim % 128 == 0 ? 128 : kv_dim;
  kpx_kv_layout lay = detail::contiguous_layout(detail::kpx_dtype(key_cache), kv_dim, hs);
  detail::report(kpx_append(detail::layer_base(key_cache, layer_idx, max_seq_len, kv_dim),
                            detail::layer_base(value_cache, layer_idx, max_seq_len, kv_dim), &lay,
                            key_out.ptr<uint8_t>(), value_out.ptr<uint8_t>(), nullptr, nullptr, start_pos,
                            seq_len, stream), "fused_kv_cache_update_cu");
}

// ---- RoPE --------------------------------------------------------------------------------
namespace detail {
inline void rope(int32_t dim, int32_t kv_dim, int32_t head_size, const tensor::Tensor& q, const tensor::Tensor& k,
                 const int32_t* positions_dev, int32_t pos_base, int32_t n, const tensor::Tensor& sin_cache,
                 const tensor::Tensor& cos_cache, void* stream, const char* what) {
  kpx_kv_layout lay = contiguous_layout(kpx_dtype(q), kv_dim, head_size);
  report(kpx_rope_append(const_cast<uint8_t*>(q.ptr<uint8_t>()), const_cast<uint8_t*>(k.ptr<uint8_t>()), nullptr,
                         dim / head_size, positions_dev, pos_base, sin_cache.ptr<float>(), cos_cache.ptr<float>(), nullptr,
                         nullptr, &lay, nullptr, n, stream), what);
}
}  // namespace detail
// input_pos must live in device memory here (the reference's CUDA path reads it on the host).
inline void rope_kernel_cu_gpu_pos(int32_t dim, int32_t kv_dim, int32_t head_size, const tensor::Tensor& input_q,
                                   const tensor::Tensor& input_k, const int32_t* pos_ptr,
                                   const tensor::Tensor& sin_cache, const tensor::Tensor& cos_cache, void* stream) {
  detail::rope(dim, kv_dim, head_size, input_q, input_k, pos_ptr, 0, 1, sin_cache, cos_cache, stream,
               "rope_kernel_cu_gpu_pos");
}
inline void rope_kernel_cu_fp16_gpu_pos(int32_t dim, int32_t kv_dim, int32_t head_size,
                                        const tensor::Tensor& input_q, const tensor::Tensor& input_k,
                                        const int32_t* pos_ptr, const tensor::Tensor& sin_cache,
                                        const tensor::Tensor& cos_cache, void* stream) {
  detail::rope(dim, kv_dim, head_size, input_q, input_k, pos_ptr, 0, 1, sin_cache, cos_cache, stream,
               "rope_kernel_cu_fp16_gpu_pos");
}
inline void rope_kernel_cu(int32_t dim, int32_t kv_dim, int32_t head_size, const tensor::Tensor& input_q,
                           const tensor::Tensor& input_k, const tensor::Tensor& input_pos,
                           const tensor::Tensor& sin_cache, const tensor::Tensor& cos_cache, void* stream) {
  const int32_t* pos = input_pos.ptr<int32_t>();
  if (input_pos.device_type() != base::DeviceType::kDeviceCUDA) {
    detail::report(KPX_ERR_INVALID_ARGUMENT, "rope_kernel_cu: the position tensor must be in device memory");
    return;
  }
  detail::rope(dim, kv_dim, head_size, input_q, input_k, pos, 0, 1, sin_cache, cos_cache, stream, "rope_kernel_cu");
}
// Batched RoPE for prefill: row s of q/k sits at position start_pos + s.
inline void batched_rope_kernel_cu(int32_t start_pos, int32_t seq_len, int32_t dim, int32_t kv_dim,
                                   int32_t head_size, const tensor::Tensor& input_q, const tensor::Tensor& input_k,
                                   const tensor::Tensor& sin_cache, const tensor::Tensor& cos_cache, void* stream) {
  detail::rope(dim, kv_dim, head_size, input_q, input_k, nullptr, start_pos, seq_len, sin_cache, cos_cache, stream,
               "batched_rope_kernel_cu");
}
inline void sin_cos_cache_calc_cu(int head_size, int max_seq_len, const tensor::Tensor& sin_cache,
                                  const tensor::Tensor& cos_cache, cudaStream_t stream, float theta = 1000000.0f) {
  detail::report(kpx_sin_cos_cache(const_cast<float*>(sin_cache.ptr<float>()), const_cast<float*>(cos_cache.ptr<float>()),
                                   head_size, max_seq_len, theta, stream), "sin_cos_cache_calc_cu");
}

}  // namespace kernel
#endif  // KUIPER_OP_KERNELS_CUDA_KV_PATH_KERNELS_H_
