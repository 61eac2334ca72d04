// Chunked-prefill attention over the paged cache.
//
// Two paths share the entry point:
//   * per-query streaming: every query token is run as a single-query attention over its
//     sequence's block-table row with length start_pos + i + 1 (the structure of the
//     reference's one-CTA-per-query prefill kernels, on the split-KV decode kernel).  Exact
//     for every dtype and size; K/V traffic grows with queries x keys.
//   * tensor-core tiles (16-bit caches): see kpx_prefill_tc.cu.
#include <vector>

#include "kpx_common.cuh"

namespace kpx {
int prefill_tc(void* out, const void* q, const void* k_pool, const void* v_pool, const kpx_kv_layout* layout,
               const int32_t* block_table, int32_t max_blocks_per_seq, const int32_t* cu_q_lens_host,
               const int32_t* start_pos_host, int32_t batch, int32_t num_q_heads, float scale, void* tile_area,
               int64_t tile_area_bytes, int32_t* status, cudaStream_t stream);
int64_t prefill_tc_area_bytes(int32_t total_q, int32_t num_q_heads);
namespace {

// 0 = tensor-core tiles where the layout allows, else per-query streaming; 1 = always streaming
int g_prefill_path = 0;

constexpr int kHeaderBytes = 256;

// lens[t] = start_pos[b] + (t - cu[b]) + 1, rows[t] = b for the query rows of sequence b
__global__ void expand_queries_kernel(const int32_t* __restrict__ cu, const int32_t* __restrict__ start,
                                      int32_t batch, int32_t total_q, int32_t* __restrict__ lens,
                                      int32_t* __restrict__ rows) {
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < total_q; t += gridDim.x * blockDim.x) {
    int lo = 0, hi = batch;  // last b with cu[b] <= t
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    lens[t] = start[lo] + (t - cu[lo]) + 1;
    rows[t] = lo;
  }
}

inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

}  // namespace
}  // namespace kpx

using namespace kpx;

extern "C" __attribute__((visibility("default"))) void kpx_internal_set_prefill_path(int v) {
  g_prefill_path = v;
}

static int64_t tile_area_bytes(int32_t total_q, int32_t num_q_heads) { return prefill_tc_area_bytes(total_q, num_q_heads); }

extern "C" int64_t kpx_prefill_workspace_bytes(int32_t total_q, int32_t num_q_heads,
                                               int32_t num_kv_heads, int32_t head_size) {
  if (total_q < 0) return -1;
  int64_t dec = kpx_decode_workspace_bytes(total_q, num_q_heads, num_kv_heads, head_size);
  if (dec < 0) return -1;
  // decode workspace, then lens[total_q], rows[total_q], cu[<=total_q+1], start[<=total_q]
  return dec + align256(int64_t(total_q) * 4) * 2 + align256((int64_t(total_q) + 1) * 4) * 2 +
         tile_area_bytes(total_q, num_q_heads);  // + work list of the tensor-core path
}

extern "C" int kpx_paged_prefill(void* out, const void* q, const void* k_pool, const void* v_pool,
                                 const kpx_kv_layout* layout, const int32_t* block_table,
                                 int32_t max_blocks_per_seq, const int32_t* cu_q_lens_host,
                                 const int32_t* start_pos_host, int32_t batch, int32_t num_q_heads,
                                 float scale, void* workspace, int64_t workspace_bytes,
                                 void* stream) {
  if (!layout_ok(layout) || !cu_q_lens_host || !start_pos_host || batch < 0 || !workspace)
    return KPX_ERR_INVALID_ARGUMENT;
  // everything both device paths dereference or store 16 bytes at a time is checked here, on
  // the host, so that a bad argument is an error code and never a device fault
  if (!out || !q || !k_pool || !v_pool || num_q_heads <= 0 || num_q_heads % layout->num_kv_heads)
    return KPX_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(q) |
       reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool) |
       reinterpret_cast<uintptr_t>(workspace)) & 15)
    return KPX_ERR_INVALID_ARGUMENT;
  if (block_table && max_blocks_per_seq <= 0) return KPX_ERR_INVALID_ARGUMENT;
  if (batch == 0) return KPX_OK;
  if (cu_q_lens_host[0] != 0) return KPX_ERR_INVALID_ARGUMENT;
  for (int32_t b = 0; b < batch; ++b)
    if (cu_q_lens_host[b + 1] < cu_q_lens_host[b] || start_pos_host[b] < 0)
      return KPX_ERR_INVALID_ARGUMENT;
  const int32_t total_q = cu_q_lens_host[batch];
  if (batch > total_q && total_q > 0) return KPX_ERR_INVALID_ARGUMENT;  // sequences without queries
  if (block_table) {
    // the last position a sequence attends to must lie inside its table row
    for (int32_t b = 0; b < batch; ++b) {
      const int64_t end = int64_t(start_pos_host[b]) + (cu_q_lens_host[b + 1] - cu_q_lens_host[b]);
      if ((end + layout->block_size - 1) / layout->block_size > max_blocks_per_seq)
        return KPX_ERR_INVALID_ARGUMENT;
    }
  }
  if (total_q == 0) return KPX_OK;
  const int64_t need = kpx_prefill_workspace_bytes(total_q, num_q_heads, layout->num_kv_heads,
                                                   layout->head_size);
  if (need < 0) return KPX_ERR_UNIMPLEMENTED;
  if (workspace_bytes < need) return KPX_ERR_WORKSPACE_TOO_SMALL;
  if (!device_info().ok) return KPX_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t dec = kpx_decode_workspace_bytes(total_q, num_q_heads, layout->num_kv_heads,
                                                 layout->head_size);
  uint8_t* base = static_cast<uint8_t*>(workspace) + dec;
  int32_t* lens = reinterpret_cast<int32_t*>(base);
  int32_t* rows = reinterpret_cast<int32_t*>(base + align256(int64_t(total_q) * 4));
  int32_t* cu = reinterpret_cast<int32_t*>(base + 2 * align256(int64_t(total_q) * 4));
  int32_t* start = reinterpret_cast<int32_t*>(base + 2 * align256(int64_t(total_q) * 4) +
                                              align256((int64_t(total_q) + 1) * 4));
  if (g_prefill_path == 0) {
    uint8_t* tile_area = base + 2 * align256(int64_t(total_q) * 4) + 2 * align256((int64_t(total_q) + 1) * 4);
    int rc = prefill_tc(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, cu_q_lens_host,
                        start_pos_host, batch, num_q_heads, scale, tile_area,
                        tile_area_bytes(total_q, num_q_heads), static_cast<int32_t*>(workspace), s);
    if (rc != KPX_ERR_UNIMPLEMENTED) return rc;
  }
  KPX_CUDA_TRY(cudaMemcpyAsync(cu, cu_q_lens_host, size_t(batch + 1) * 4, cudaMemcpyHostToDevice, s));
  KPX_CUDA_TRY(cudaMemcpyAsync(start, start_pos_host, size_t(batch) * 4, cudaMemcpyHostToDevice, s));
  expand_queries_kernel<<<(total_q + 255) / 256, 256, 0, s>>>(cu, start, batch, total_q, lens, rows);
  KPX_CUDA_TRY(cudaGetLastError());
  (void)kHeaderBytes;
  return decode_rows(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, rows, lens, 0,
                     total_q, num_q_heads, scale, workspace, dec, stream);
}
