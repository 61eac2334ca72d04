// Entry points of the paged GQA decode attention (kernel and launch forms: kpx_decode_impl.cuh;
// the kernels themselves are instantiated per element type in kpx_decode_{f16,bf16,f32}.cu).
#include <climits>

#include "kpx_decode_impl.cuh"

namespace kpx {
namespace decode {
// Tuning knob: 0 = default shape; set through kpx_internal_set_decode_variant.
int g_decode_variant = 0;
// Small launches (see paged_decode_kernel): used when batch x table width x items per sequence
// is below g_small_below blocks per warp of the grid; then ranges hold at least
// g_min_blocks_per_range blocks while at least g_min_warps_per_sm warps per SM stay active.
int g_small_below = 12, g_min_blocks_per_range = 12, g_min_warps_per_sm = 4;
// Test-only: polls before a bounded wait gives up, and the warp whose first tile never comes.
uint32_t g_wait_limit = kWaitLimit;
int g_withhold_worker = -1;
}  // namespace decode
}  // namespace kpx

using namespace kpx;
using namespace kpx::decode;

extern "C" __attribute__((visibility("default"))) void kpx_internal_set_decode_variant(int v) {
  g_decode_variant = v;
}
extern "C" __attribute__((visibility("default"))) void kpx_internal_set_decode_small(int below, int min_blocks,
                                                                                       int min_warps) {
  g_small_below = below;
  if (min_blocks > 0) g_min_blocks_per_range = min_blocks;
  if (min_warps >= 0) g_min_warps_per_sm = min_warps;
}

// Not in the header: lets a test make a bounded wait run out (the tile request of one warp is
// announced but never issued; every other warp finishes) without a faulting or endless kernel.
extern "C" __attribute__((visibility("default"))) void kpx_internal_set_decode_fault(uint32_t wait_limit,
                                                                                       int withhold_worker) {
  g_wait_limit = wait_limit ? wait_limit : kWaitLimit;
  g_withhold_worker = withhold_worker;
}

namespace {
constexpr int64_t kSlotBytes = (4 * kD + 8) * sizeof(float);
// (the built-in scratch of kpx_paged_decode_static is this size for its head-layout limit)
int64_t min_workspace_bytes(int32_t num_q_heads, int32_t num_kv_heads) {
  return int64_t(kStatusBytes) + counter_bytes(num_q_heads, num_kv_heads) + int64_t(kMinPartialSlots) * kSlotBytes;
}
}  // namespace

extern "C" int64_t kpx_decode_workspace_bytes(int32_t batch, int32_t num_q_heads,
                                              int32_t num_kv_heads, int32_t head_size) {
  (void)batch;
  if (num_q_heads <= 0 || num_kv_heads <= 0 || head_size != kD || num_q_heads % num_kv_heads)
    return -1;
  // header + one counter per item of a launch + 2 partial slots per persistent warp,
  // each up to 4 heads x (128 + 2) floats
  return min_workspace_bytes(num_q_heads, num_kv_heads);
}

extern "C" int kpx_paged_decode(void* out, const void* q, const void* k_pool, const void* v_pool,
                                const kpx_kv_layout* layout, const int32_t* block_table,
                                int32_t max_blocks_per_seq, const int32_t* seq_lens,
                                int32_t len_bias, int32_t batch, int32_t num_q_heads, float scale,
                                void* workspace, int64_t workspace_bytes, void* stream) {
  return kpx::decode_rows(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, nullptr,
                          seq_lens, len_bias, batch, num_q_heads, scale, workspace, workspace_bytes,
                          stream);
}

extern "C" int kpx_paged_decode_overlapped(void* out, const void* q, const void* k_pool, const void* v_pool,
                                           const kpx_kv_layout* layout, const int32_t* block_table,
                                           int32_t max_blocks_per_seq, const int32_t* seq_lens,
                                           int32_t len_bias, int32_t batch, int32_t num_q_heads, float scale,
                                           void* workspace, int64_t workspace_bytes, void* stream) {
  return kpx::decode_rows(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, nullptr,
                          seq_lens, len_bias, batch, num_q_heads, scale, workspace, workspace_bytes,
                          stream, nullptr, KPX_DECODE_OVERLAPPED);
}

// ---------------------------------------------------------------------------------------
// Plan of a decode step (layout: kpx_decode_impl.cuh).
namespace kpx {
namespace {
constexpr int kPlanThreads = 128;
// One thread per warp of the decode launch: where its range of the line of blocks starts.
__global__ void __launch_bounds__(kPlanThreads) decode_plan_kernel(const DecodeParams p, int32_t* plan, int workers) {
  __shared__ int prefix[kMaxBatch + 1];
  __shared__ int bad;
  const int tid = threadIdx.x;
  if (tid == 0) bad = 0;
  for (int b = tid; b < p.batch; b += kPlanThreads) {
    prefix[b + 1] = blocks_of(seq_len_of(p, b));
    if (p.block_table && p.seq_lens && p.seq_lens[b] + p.len_bias > p.max_cached_tokens) bad = 1;
  }
  if (tid == 0) prefix[0] = 0;
  __syncthreads();
  if (tid < 32) {  // inclusive scan in chunks of 32
    int carry = 0;
    for (int base = 0; base < p.batch; base += 32) {
      const int i = base + tid;
      int v = i < p.batch ? prefix[i + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, d);
        if (tid >= d) v += n;
      }
      if (i < p.batch) prefix[i + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int b = tid; b <= p.batch; b += kPlanThreads) plan[kPlanPrefixAt + b] = prefix[b];
    if (tid == 0) {
      plan[1] = p.batch;
      plan[2] = workers;
      plan[3] = p.num_kv_heads * p.head_groups;
      plan[4] = bad ? KPX_ERR_INVALID_ARGUMENT : 0;
      __threadfence();
      plan[0] = kPlanMark;
    }
  }
  const int w = blockIdx.x * kPlanThreads + tid;
  if (w >= workers) return;
  // the cut of the line and the search are the decode kernel's own (Split, Cursor::locate)
  const int64_t total = int64_t(prefix[p.batch]) * p.num_kv_heads * p.head_groups;
  Split split;
  split.quot = total / workers;
  split.rem = total - split.quot * workers;
  const int64_t u0 = split.start(w), u1 = split.start(w + 1);
  int4 e = make_int4(0xffff << 16, 0, 0, 0);
  if (u0 < u1) {
    Cursor cur;
    cur.locate(p, prefix, u0);
    e.x = (cur.b << 16) | cur.sub;
    e.y = cur.blk;
    e.z = cur.len;
    e.w = cur.row ? cur.row[cur.blk] : cur.blk;
  }
  reinterpret_cast<int4*>(plan + kPlanEntriesAt)[w] = e;
}
}  // namespace
}  // namespace kpx

extern "C" int64_t kpx_decode_plan_bytes(void) {
  return int64_t(kPlanEntriesAt + kMaxSms * kMaxWarpsPerCta * kPlanEntryWords) * 4;
}

extern "C" int kpx_decode_plan(void* plan, int64_t plan_bytes, const kpx_kv_layout* layout,
                               const int32_t* block_table, int32_t max_blocks_per_seq, const int32_t* seq_lens,
                               int32_t len_bias, int32_t batch, int32_t num_q_heads, void* stream) {
  if (!layout_ok(layout) || !plan || (reinterpret_cast<uintptr_t>(plan) & 15) || batch < 0 || num_q_heads <= 0)
    return KPX_ERR_INVALID_ARGUMENT;
  if (plan_bytes < kpx_decode_plan_bytes()) return KPX_ERR_WORKSPACE_TOO_SMALL;
  if (layout->head_size != kD || layout->block_size != kBS) return KPX_ERR_UNIMPLEMENTED;
  if (num_q_heads % layout->num_kv_heads) return KPX_ERR_INVALID_ARGUMENT;
  if (block_table && max_blocks_per_seq <= 0) return KPX_ERR_INVALID_ARGUMENT;
  if (!seq_lens && len_bias < 0) return KPX_ERR_INVALID_ARGUMENT;
  if (!device_info().ok) return KPX_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (batch == 0 || batch > kMaxBatch) {
    // nothing to plan, or a batch that decode serves in slices: a plan without its mark is ignored
    return cuda_status(cudaMemsetAsync(plan, 0, 32, s));
  }
  DecodeParams p{};
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.row_index = nullptr;
  p.max_blocks_per_seq = max_blocks_per_seq;
  {
    const int64_t row_tokens = int64_t(max_blocks_per_seq) * kBS;
    p.max_cached_tokens = block_table ? int32_t(row_tokens > INT32_MAX ? INT32_MAX : row_tokens) : 0;
  }
  p.len_bias = len_bias;
  p.batch = batch;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = layout->num_kv_heads;
  p.kv_mul = num_q_heads / layout->num_kv_heads;
  const int qh = heads_per_warp(p.kv_mul);
  p.head_groups = (p.kv_mul + qh - 1) / qh;
  // the warps of the launch forms that take a plan: 12 per SM for 16-bit caches (one CTA of 12
  // or three of 4), 6 for fp32
  int sms = device_info().sm_count;
  if (sms > kMaxSms) sms = kMaxSms;
  const int workers = sms * (layout->dtype == KPX_F32 ? 6 : 12);
  decode_plan_kernel<<<(workers + kPlanThreads - 1) / kPlanThreads, kPlanThreads, 0, s>>>(
      p, static_cast<int32_t*>(plan), workers);
  return cuda_status(cudaGetLastError());
}

extern "C" int kpx_paged_decode_planned(void* out, const void* q, const void* k_pool, const void* v_pool,
                                        const kpx_kv_layout* layout, const int32_t* block_table,
                                        int32_t max_blocks_per_seq, const int32_t* seq_lens, int32_t len_bias,
                                        int32_t batch, int32_t num_q_heads, float scale, void* workspace,
                                        int64_t workspace_bytes, const void* plan, int32_t flags, void* stream) {
  if (flags & ~KPX_DECODE_OVERLAPPED) return KPX_ERR_INVALID_ARGUMENT;
  if (plan && (reinterpret_cast<uintptr_t>(plan) & 15)) return KPX_ERR_INVALID_ARGUMENT;
  return kpx::decode_rows(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, nullptr,
                          seq_lens, len_bias, batch, num_q_heads, scale, workspace, workspace_bytes,
                          stream, nullptr, flags, plan);
}

extern "C" int kpx_rope_append_decode(void* out, const void* q, const void* k_new, const void* v_new,
                                      const float* sin_cache, const float* cos_cache, void* k_pool,
                                      void* v_pool, const kpx_kv_layout* layout,
                                      const int32_t* block_table, int32_t max_blocks_per_seq,
                                      const int32_t* positions, int32_t batch, int32_t num_q_heads,
                                      float scale, void* workspace, int64_t workspace_bytes,
                                      int32_t flags, void* stream) {
  if (!k_new || !v_new || !sin_cache || !cos_cache || !positions) return KPX_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new) |
       reinterpret_cast<uintptr_t>(sin_cache) | reinterpret_cast<uintptr_t>(cos_cache)) & 15)
    return KPX_ERR_INVALID_ARGUMENT;
  if (flags & ~KPX_DECODE_OVERLAPPED) return KPX_ERR_INVALID_ARGUMENT;
  const kpx::FusedStep fused{k_new, v_new, sin_cache, cos_cache};
  return kpx::decode_rows(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, nullptr,
                          positions, 0, batch, num_q_heads, scale, workspace, workspace_bytes, stream,
                          &fused, flags);
}

int kpx::decode_rows(void* out, const void* q, const void* k_pool, const void* v_pool,
                     const kpx_kv_layout* layout, const int32_t* block_table,
                     int32_t max_blocks_per_seq, const int32_t* row_index, const int32_t* seq_lens,
                     int32_t len_bias, int32_t batch, int32_t num_q_heads, float scale,
                     void* workspace, int64_t workspace_bytes, void* stream, const FusedStep* fused,
                     int flags, const void* plan) {
  if (!layout_ok(layout) || !out || !q || !k_pool || !v_pool || batch < 0 || num_q_heads <= 0)
    return KPX_ERR_INVALID_ARGUMENT;
  if (layout->head_size != kD || layout->block_size != kBS) return KPX_ERR_UNIMPLEMENTED;
  if (num_q_heads % layout->num_kv_heads) return KPX_ERR_INVALID_ARGUMENT;
  if (num_q_heads / layout->num_kv_heads > 64) return KPX_ERR_UNIMPLEMENTED;
  if (block_table && max_blocks_per_seq <= 0) return KPX_ERR_INVALID_ARGUMENT;
  if (!seq_lens && len_bias < 0) return KPX_ERR_INVALID_ARGUMENT;
  if (!seq_lens && block_table && int64_t(len_bias) > int64_t(max_blocks_per_seq) * kBS)
    return KPX_ERR_INVALID_ARGUMENT;  // a fixed length the table rows cannot hold
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15)) return KPX_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool) |
       reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15)
    return KPX_ERR_INVALID_ARGUMENT;
  if (kpx_decode_workspace_bytes(batch, num_q_heads, layout->num_kv_heads, layout->head_size) < 0)
    return KPX_ERR_UNIMPLEMENTED;
  if (workspace_bytes < min_workspace_bytes(num_q_heads, layout->num_kv_heads)) return KPX_ERR_WORKSPACE_TOO_SMALL;
  if (batch == 0) return KPX_OK;
  if (!device_info().ok) return KPX_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int eb = elt_bytes(layout->dtype);
  DecodeParams p;
  p.k_pool = static_cast<const uint8_t*>(k_pool);
  p.v_pool = static_cast<const uint8_t*>(v_pool);
  p.k_new = fused ? fused->k_new : nullptr;
  p.v_new = fused ? fused->v_new : nullptr;
  p.sin_cache = fused ? fused->sin_cache : nullptr;
  p.cos_cache = fused ? fused->cos_cache : nullptr;
  p.k_pool_w = fused ? static_cast<uint8_t*>(const_cast<void*>(k_pool)) : nullptr;
  p.v_pool_w = fused ? static_cast<uint8_t*>(const_cast<void*>(v_pool)) : nullptr;
  p.status = static_cast<int32_t*>(workspace);
  p.counters = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) + kStatusBytes);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kStatusBytes +
                                        counter_bytes(num_q_heads, layout->num_kv_heads));
  p.block_stride_b = layout->block_stride * eb;
  p.head_stride_b = layout->head_stride * eb;
  p.token_stride_b = layout->token_stride * eb;
  p.num_blocks = layout->num_blocks;
  p.max_blocks_per_seq = max_blocks_per_seq;
  // the fused step stores its new token at position len: the row must hold one more
  {
    const int64_t row_tokens = int64_t(max_blocks_per_seq) * kBS - (fused ? 1 : 0);
    p.max_cached_tokens = block_table ? int32_t(row_tokens > INT32_MAX ? INT32_MAX : row_tokens) : 0;
  }
  p.len_bias = len_bias;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = layout->num_kv_heads;
  p.kv_mul = num_q_heads / layout->num_kv_heads;
  p.head_groups = 1;
  p.partial_slots = kMinPartialSlots;
  p.tile_contig = tile_contiguous(layout) ? 1 : 0;
  p.min_blocks_per_range = g_min_blocks_per_range;
  p.min_warps_per_sm = g_min_warps_per_sm;
  p.wait_limit = g_wait_limit;
  p.withhold_worker = g_withhold_worker;
  p.qscale = scale * kLog2e;
  // a plan covers one launch of the whole batch as it is (no slices, no row indirection)
  p.plan = (plan && batch <= kMaxBatch && !row_index && !fused) ? static_cast<const int32_t*>(plan) : nullptr;
  // the block prefix of one launch lives in shared memory: long batches go in slices
  for (int32_t b0 = 0; b0 < batch; b0 += kMaxBatch) {
    int32_t nb = batch - b0 < kMaxBatch ? batch - b0 : kMaxBatch;
    p.batch = nb;
    p.out = static_cast<uint8_t*>(out) + int64_t(b0) * num_q_heads * kD * eb;
    p.q = static_cast<const uint8_t*>(q) + int64_t(b0) * num_q_heads * kD * eb;
    p.row_index = row_index ? row_index + b0 : nullptr;
    p.block_table = (block_table && !row_index) ? block_table + int64_t(b0) * max_blocks_per_seq
                                                : block_table;
    p.seq_lens = seq_lens ? seq_lens + b0 : nullptr;
    if (fused) {
      p.k_new = static_cast<const uint8_t*>(fused->k_new) + int64_t(b0) * layout->num_kv_heads * kD * eb;
      p.v_new = static_cast<const uint8_t*>(fused->v_new) + int64_t(b0) * layout->num_kv_heads * kD * eb;
    }
    int rc;
    switch (layout->dtype) {
      case KPX_F16: rc = dispatch_decode<__half>(p, s, flags); break;
      case KPX_BF16: rc = dispatch_decode<__nv_bfloat16>(p, s, flags); break;
      default: rc = dispatch_decode<float>(p, s, flags); break;
    }
    if (rc != KPX_OK) return rc;
  }
  return KPX_OK;
}

// ---------------------------------------------------------------------------------------
// Decode without a caller-provided workspace.
//
// Some callers cannot hand over scratch memory: a plugin running inside a host that owns
// the whole device heap, code on a stream whose owner forbids cudaMalloc between steps, a
// kernel registry that only passes inputs and outputs.  For them the scratch of
// kpx_paged_decode (status word, per-item piece counters, split-KV partials) lives in the
// array below: file-scope device memory that every GPU loading this library holds until
// the process exits.
namespace kpx {
namespace {
constexpr int kStaticMaxItemsPerSeq = 16;  // num_kv_heads * head groups, e.g. 8 KV heads x 8 query heads each
constexpr int64_t kStaticCounterBytes = 65536;  // >= kMaxBatch * kStaticMaxItemsPerSeq counters
static_assert(int64_t(kMaxBatch) * kStaticMaxItemsPerSeq * 4 <= kStaticCounterBytes, "counter area");
constexpr int64_t kStaticScratchBytes =
    kStatusBytes + kStaticCounterBytes + int64_t(kMinPartialSlots) * kSlotBytes;  // 10 715 392 bytes
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
}  // namespace
}  // namespace kpx

extern "C" int kpx_paged_decode_static(void* out, const void* q, const void* k_pool,
                                       const void* v_pool, const kpx_kv_layout* layout,
                                       const int32_t* block_table, int32_t max_blocks_per_seq,
                                       const int32_t* seq_lens, int32_t len_bias, int32_t batch,
                                       int32_t num_q_heads, float scale, void* stream) {
  if (!layout_ok(layout) || num_q_heads <= 0 || num_q_heads % layout->num_kv_heads)
    return KPX_ERR_INVALID_ARGUMENT;
  const int kv_mul = num_q_heads / layout->num_kv_heads;
  const int qh = heads_per_warp(kv_mul);
  const int per_seq = layout->num_kv_heads * ((kv_mul + qh - 1) / qh);
  if (per_seq > kStaticMaxItemsPerSeq) return KPX_ERR_STATIC_SCRATCH_LIMIT;
  if (kpx_decode_workspace_bytes(batch, num_q_heads, layout->num_kv_heads, layout->head_size) < 0)
    return KPX_ERR_UNIMPLEMENTED;
  if (min_workspace_bytes(num_q_heads, layout->num_kv_heads) > kStaticScratchBytes)
    return KPX_ERR_STATIC_SCRATCH_LIMIT;
  if (!device_info().ok) return KPX_ERR_CUDA;
  // In host code `g_static_scratch` names a host-side stand-in, not device memory: the
  // address a kernel may use comes from cudaGetSymbolAddress, asked once per device with
  // that device current.
  static void* scratch_of_device[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  KPX_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return KPX_ERR_CUDA;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!scratch_of_device[dev]) {
      void* ptr = nullptr;
      if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) {
        (void)cudaGetLastError();
        return KPX_ERR_CUDA;
      }
      scratch_of_device[dev] = ptr;
    }
    scratch = scratch_of_device[dev];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left: the status word and the piece
  // counters must start at zero (partials are always written before they are read).
  KPX_CUDA_TRY(cudaMemsetAsync(scratch, 0, size_t(kStatusBytes + kStaticCounterBytes), s));
  {
    // the group counters of the two-level assembly live in the last partial slot
    const int qh = heads_per_warp(num_q_heads / layout->num_kv_heads);
    const size_t slot_bytes = size_t(qh * kD + 8) * sizeof(float);
    uint8_t* partials = static_cast<uint8_t*>(scratch) + kStatusBytes + counter_bytes(num_q_heads, layout->num_kv_heads);
    KPX_CUDA_TRY(cudaMemsetAsync(partials + size_t(kMinPartialSlots - 1) * slot_bytes, 0, slot_bytes, s));
  }
  return kpx_paged_decode(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq,
                          seq_lens, len_bias, batch, num_q_heads, scale, scratch,
                          kStaticScratchBytes, stream);
}
