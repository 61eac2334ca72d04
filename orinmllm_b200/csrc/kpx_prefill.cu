// Chunked-prefill attention over the paged cache (placeholder entry points; the
// kernel lands in this file).
#include "kpx_common.cuh"

extern "C" int64_t kpx_prefill_workspace_bytes(int32_t total_q, int32_t num_q_heads,
                                               int32_t num_kv_heads, int32_t head_size) {
  (void)total_q; (void)num_q_heads; (void)num_kv_heads; (void)head_size;
  return 256;
}

extern "C" int kpx_paged_prefill(void*, const void*, const void*, const void*, const kpx_kv_layout*,
                                 const int32_t*, int32_t, const int32_t*, const int32_t*, int32_t,
                                 int32_t, float, void*, int64_t, void*) {
  return KPX_ERR_UNIMPLEMENTED;
}
