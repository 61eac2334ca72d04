// K/V append into the block pool, RoPE(+append), sin/cos tables, copy-on-write
// block copy and block refcount updates.  All of these are pure data movement
// (or element-wise fp32 math) bound by HBM bandwidth: 128-bit accesses,
// grid-stride loops sized from the SM count.
#include "kpx_common.cuh"

namespace kpx {
namespace {

struct LayoutDev {
  int64_t block_stride, head_stride, token_stride;  // elements
  int32_t num_kv_heads, head_size, block_size, elt_bytes;
};

inline LayoutDev to_dev(const kpx_kv_layout* l) {
  LayoutDev d;
  d.block_stride = l->block_stride;
  d.head_stride = l->head_stride;
  d.token_stride = l->token_stride;
  d.num_kv_heads = l->num_kv_heads;
  d.head_size = l->head_size;
  d.block_size = l->block_size;
  d.elt_bytes = elt_bytes(l->dtype);
  return d;
}

// Byte offset of element 0 of (slot, head) in a pool.
__device__ __forceinline__ int64_t slot_head_offset_bytes(const LayoutDev& L, int64_t slot, int h) {
  int64_t blk = slot / L.block_size;
  int64_t off = slot - blk * L.block_size;
  return (blk * L.block_stride + int64_t(h) * L.head_stride + off * L.token_stride) * L.elt_bytes;
}

// token index and remainder of work item i (32-bit division whenever the item count allows it)
__device__ __forceinline__ void split_item(int64_t i, int per_tok, bool small, int64_t& t, int& r) {
  if (small) {
    const uint32_t q = uint32_t(i) / uint32_t(per_tok);
    t = q;
    r = int(uint32_t(i) - q * uint32_t(per_tok));
  } else {
    t = i / per_tok;
    r = int(i - t * per_tok);
  }
}
__device__ __forceinline__ int64_t slot_head_offset_bytes_fast(const LayoutDev& L, int64_t slot, int h) {
  int64_t blk, off;
  if (uint64_t(slot) < 0x80000000ull) {
    const uint32_t b = uint32_t(slot) / uint32_t(L.block_size);
    blk = b;
    off = uint32_t(slot) - b * uint32_t(L.block_size);
  } else {
    blk = slot / L.block_size;
    off = slot - blk * L.block_size;
  }
  return (blk * L.block_stride + int64_t(h) * L.head_stride + off * L.token_stride) * L.elt_bytes;
}

// One thread moves kAppendUnroll 16-byte vectors of K or V per step of the grid-stride loop:
// all of a step's loads are issued before its first store, so that a thread keeps several
// loads in flight (one at a time leaves about 32 KB per SM in flight, short of what the
// memory system needs to run at full rate).
constexpr int kAppendUnroll = 4;
__global__ void __launch_bounds__(256)
append_kernel(uint8_t* __restrict__ k_pool, uint8_t* __restrict__ v_pool,
              const uint8_t* __restrict__ k_src, const uint8_t* __restrict__ v_src,
              const int64_t* __restrict__ slot_mapping, const int32_t* __restrict__ pos_dev,
              int32_t pos_bias, int32_t num_tokens, LayoutDev L) {
  const int vec_per_head = L.head_size * L.elt_bytes / 16;
  const int vec_per_tok = vec_per_head * L.num_kv_heads;
  const int which_n = v_pool ? 2 : 1;
  const int per_tok = vec_per_tok * which_n;
  const int64_t total = int64_t(num_tokens) * per_tok;
  const bool small = total < (int64_t(1) << 31);
  int64_t base_slot = 0;
  if (!slot_mapping) base_slot = int64_t(pos_dev ? *pos_dev : 0) + pos_bias;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i0 = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i0 < total; i0 += stride * kAppendUnroll) {
    uint4 val[kAppendUnroll];
    uint8_t* dst[kAppendUnroll];
#pragma unroll
    for (int u = 0; u < kAppendUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      dst[u] = nullptr;
      if (i >= total) continue;
      int64_t t;
      int r;
      split_item(i, per_tok, small, t, r);
      const int which = r >= vec_per_tok ? 1 : 0;
      const int vec = r - which * vec_per_tok;
      const int h = vec / vec_per_head;
      const int vi = vec - h * vec_per_head;
      // the source row exists whatever the slot says: its load does not wait for the slot's
      val[u] = __ldg(reinterpret_cast<const uint4*>((which ? v_src : k_src) + (t * vec_per_tok + vec) * 16));
      const int64_t slot = slot_mapping ? slot_mapping[t] : base_slot + t;
      if (slot < 0) continue;
      dst[u] = (which ? v_pool : k_pool) + slot_head_offset_bytes_fast(L, slot, h) + vi * 16;
    }
#pragma unroll
    for (int u = 0; u < kAppendUnroll; ++u)
      if (dst[u]) *reinterpret_cast<uint4*>(dst[u]) = val[u];
  }
}

// RoPE in place on Q and K rows, then optional append of the rotated K and of V.
// One thread owns one rotation pair-group: 8 (16-bit) or 4 (fp32) consecutive j
// of one head of one token, i.e. one 16-byte vector at j and one at j+head_size/2.
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ q, T* __restrict__ k, const T* __restrict__ v,
                                   int32_t q_heads, const int32_t* __restrict__ positions,
                                   int32_t pos_base, const float* __restrict__ sin_cache,
                                   const float* __restrict__ cos_cache, uint8_t* __restrict__ k_pool,
                                   uint8_t* __restrict__ v_pool,
                                   const int64_t* __restrict__ slot_mapping, int32_t num_tokens,
                                   LayoutDev L, const float* __restrict__ q_norm_w,
                                   const float* __restrict__ k_norm_w, float norm_eps) {
  constexpr int E = Elt<T>::kPer16B;
  const int hs = L.head_size;
  const int groups_per_head = hs / 2 / E;  // pair-groups per head
  const int kvh = L.num_kv_heads;
  const int heads_qk = (q ? q_heads : 0) + (k ? kvh : 0);
  const int vvec_per_tok = (v && v_pool) ? kvh * hs / E : 0;
  const int work_per_tok = heads_qk * groups_per_head + vvec_per_tok;
  const int64_t total = int64_t(num_tokens) * work_per_tok;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    int64_t t = i / work_per_tok;
    int r = int(i - t * work_per_tok);
    int64_t slot = slot_mapping ? slot_mapping[t] : -1;
    if (r >= heads_qk * groups_per_head) {
      // plain V copy into the pool
      if (slot < 0) continue;
      int vec = r - heads_qk * groups_per_head;
      int h = vec / (hs / E);
      int vi = vec - h * (hs / E);
      const uint4* src = reinterpret_cast<const uint4*>(v + (t * kvh + h) * int64_t(hs)) + vi;
      *reinterpret_cast<uint4*>(v_pool + slot_head_offset_bytes(L, slot, h) + vi * 16) = __ldg(src);
      continue;
    }
    int head = r / groups_per_head;
    int g = r - head * groups_per_head;
    bool is_k = q ? head >= q_heads : true;
    int h = is_k ? head - (q ? q_heads : 0) : head;
    T* row = is_k ? k + (t * kvh + h) * int64_t(hs) : q + (t * q_heads + h) * int64_t(hs);
    const int32_t pos = (positions ? positions[t] : int32_t(t)) + pos_base;
    uint4 lo_raw = *reinterpret_cast<const uint4*>(row + g * E);
    uint4 hi_raw = *reinterpret_cast<const uint4*>(row + hs / 2 + g * E);
    float lo[E], hi[E];
    Elt<T>::unpack(lo_raw, lo);
    Elt<T>::unpack(hi_raw, hi);
    const float* norm_w = is_k ? k_norm_w : q_norm_w;
    if (norm_w) {
      // per-head RMSNorm before the rotation (Qwen3 q/k norm): the head's groups_per_head
      // threads are consecutive lanes of one warp and walk this path together
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) ss = fmaf(hi[e], hi[e], fmaf(lo[e], lo[e], ss));
      const int lane = threadIdx.x & 31;
      const uint32_t head_mask = (groups_per_head >= 32 ? 0xffffffffu : ((1u << groups_per_head) - 1u))
                                 << (lane & ~(groups_per_head - 1));
      for (int m = 1; m < groups_per_head; m <<= 1) ss += __shfl_xor_sync(head_mask, ss, m);
      const float rs = 1.f / sqrtf(ss / float(hs) + norm_eps);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        lo[e] = __ldg(norm_w + g * E + e) * (rs * lo[e]);
        hi[e] = __ldg(norm_w + hs / 2 + g * E + e) * (rs * hi[e]);
      }
    }
    __align__(16) T lo_out[E];
    __align__(16) T hi_out[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      int j = g * E + e;
      float fci = __ldg(sin_cache + int64_t(pos) * hs + 2 * j);
      float fcr = __ldg(cos_cache + int64_t(pos) * hs + 2 * j);
      // v0*cos - v1*sin and v0*sin + v1*cos with separately rounded products, as
      // the reference CPU statement computes them (no FMA contraction).
      float r0 = __fsub_rn(__fmul_rn(lo[e], fcr), __fmul_rn(hi[e], fci));
      float r1 = __fadd_rn(__fmul_rn(lo[e], fci), __fmul_rn(hi[e], fcr));
      lo_out[e] = Elt<T>::from_float(r0);
      hi_out[e] = Elt<T>::from_float(r1);
    }
    uint4 lo_w = *reinterpret_cast<uint4*>(lo_out);
    uint4 hi_w = *reinterpret_cast<uint4*>(hi_out);
    *reinterpret_cast<uint4*>(row + g * E) = lo_w;
    *reinterpret_cast<uint4*>(row + hs / 2 + g * E) = hi_w;
    if (is_k && k_pool && slot >= 0) {
      uint8_t* dst = k_pool + slot_head_offset_bytes(L, slot, h);
      *reinterpret_cast<uint4*>(dst + g * 16) = lo_w;
      *reinterpret_cast<uint4*>(dst + (hs / 2) * sizeof(T) + g * 16) = hi_w;
    }
  }
}

// ---- token-walking form of the plain append ------------------------------------------
// When a token's work items fit one CTA (<= 1024), thread r of the CTA does item r of every
// token the CTA visits (tokens blockIdx.x, blockIdx.x + gridDim.x, ...).  A thread's role
// (which head, which vector, K or V) is then fixed for the whole launch and is decoded once;
// per token there is one slot fetch and one 64-bit base address.  append_kernel above (one flat
// index per item, decoded anew each time) remains the fallback for wider tokens: it spends
// about half of the SM's issue slots on index arithmetic at 16 bytes per item.  (The same
// form of the RoPE kernel measured no faster than the flat one and is not kept.)
__device__ __forceinline__ int64_t slot_base_bytes(const LayoutDev& L, int64_t slot) {
  int64_t blk, off;
  if (uint64_t(slot) < 0x80000000ull) {
    const uint32_t b = uint32_t(slot) / uint32_t(L.block_size);
    blk = b;
    off = uint32_t(slot) - b * uint32_t(L.block_size);
  } else {
    blk = slot / L.block_size;
    off = slot - blk * L.block_size;
  }
  return (blk * L.block_stride + off * L.token_stride) * L.elt_bytes;
}

constexpr int kTokenUnroll = 4;
__global__ void __launch_bounds__(1024)
append_token_kernel(uint8_t* __restrict__ k_pool, uint8_t* __restrict__ v_pool,
                    const uint8_t* __restrict__ k_src, const uint8_t* __restrict__ v_src,
                    const int64_t* __restrict__ slot_mapping, const int32_t* __restrict__ pos_dev,
                    int32_t pos_bias, int32_t num_tokens, LayoutDev L) {
  const int vec_per_head = L.head_size * L.elt_bytes / 16;
  const int vec_per_tok = vec_per_head * L.num_kv_heads;
  const int r = threadIdx.x;
  if (r >= vec_per_tok * (v_pool ? 2 : 1)) return;
  const int which = r >= vec_per_tok ? 1 : 0;
  const int vec = r - which * vec_per_tok;
  const int h = vec / vec_per_head;
  const int vi = vec - h * vec_per_head;
  const uint8_t* src = (which ? v_src : k_src) + vec * 16;
  uint8_t* pool = (which ? v_pool : k_pool) + int64_t(h) * L.head_stride * L.elt_bytes + vi * 16;
  const int64_t src_tok_bytes = int64_t(vec_per_tok) * 16;
  int64_t base_slot = 0;
  if (!slot_mapping) base_slot = int64_t(pos_dev ? *pos_dev : 0) + pos_bias;
  for (int64_t t0 = blockIdx.x; t0 < num_tokens; t0 += int64_t(gridDim.x) * kTokenUnroll) {
    uint4 val[kTokenUnroll];
    int64_t slot[kTokenUnroll];
#pragma unroll
    for (int u = 0; u < kTokenUnroll; ++u) {
      const int64_t t = t0 + int64_t(u) * gridDim.x;
      slot[u] = -1;
      if (t >= num_tokens) continue;
      val[u] = __ldg(reinterpret_cast<const uint4*>(src + t * src_tok_bytes));
      slot[u] = slot_mapping ? slot_mapping[t] : base_slot + t;
    }
#pragma unroll
    for (int u = 0; u < kTokenUnroll; ++u)
      if (slot[u] >= 0) *reinterpret_cast<uint4*>(pool + slot_base_bytes(L, slot[u])) = val[u];
  }
}

__global__ void sin_cos_kernel(float* __restrict__ sin_cache, float* __restrict__ cos_cache,
                               int32_t head_size, int32_t max_seq_len, float theta) {
  int64_t total = int64_t(head_size) * max_seq_len;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    int pos = int(i / head_size);
    int hd = int(i - int64_t(pos) * head_size);
    float freq = 1.0f / powf(theta, float(hd) / float(head_size));
    float val = float(pos) * freq;
    sin_cache[i] = sinf(val);
    cos_cache[i] = cosf(val);
  }
}

// Copy-on-write: whole blocks, every layer, K and V.  One CTA-row of threads per
// 16-byte vector; a block's (head) tiles are copied tile by tile so both the
// paged and the strided layout work.
__global__ void cow_copy_kernel(uint8_t* __restrict__ k_pool, uint8_t* __restrict__ v_pool,
                                int32_t num_layers, int64_t layer_stride_bytes,
                                const int32_t* __restrict__ src_ids,
                                const int32_t* __restrict__ dst_ids, int32_t n, LayoutDev L) {
  const int vec_per_row = L.head_size * L.elt_bytes / 16;
  const int64_t vec_per_block = int64_t(vec_per_row) * L.block_size * L.num_kv_heads;
  const int64_t total = vec_per_block * n * num_layers * 2;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    int64_t r = i;
    int vi = int(r % vec_per_row);
    r /= vec_per_row;
    int tok = int(r % L.block_size);
    r /= L.block_size;
    int h = int(r % L.num_kv_heads);
    r /= L.num_kv_heads;
    int which = int(r & 1);
    r >>= 1;
    int layer = int(r % num_layers);
    int pair = int(r / num_layers);
    int64_t s = src_ids[pair], d = dst_ids[pair];
    if (s < 0 || d < 0 || s == d) continue;
    uint8_t* pool = (which ? v_pool : k_pool) + layer * layer_stride_bytes;
    int64_t in_block = (int64_t(h) * L.head_stride + int64_t(tok) * L.token_stride) * L.elt_bytes + vi * 16;
    const uint4* src = reinterpret_cast<const uint4*>(pool + s * L.block_stride * L.elt_bytes + in_block);
    uint4* dst = reinterpret_cast<uint4*>(pool + d * L.block_stride * L.elt_bytes + in_block);
    *dst = *src;
  }
}

__global__ void refcount_kernel(int32_t* __restrict__ refcounts, int32_t num_blocks,
                                const int32_t* __restrict__ block_ids,
                                const int32_t* __restrict__ deltas, int32_t n,
                                int32_t* __restrict__ error_count) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    int32_t b = block_ids[i];
    int32_t d = deltas[i];
    if (b < 0 || b >= num_blocks) {
      if (error_count) atomicAdd(error_count, 1);
      continue;
    }
    if (d >= 0) {
      atomicAdd(refcounts + b, d);
    } else {
      // never drive a count below zero: compare-and-swap loop (bounded by contention only)
      int32_t old = refcounts[b];
      while (true) {
        if (old + d < 0) {
          if (error_count) atomicAdd(error_count, 1);
          break;
        }
        int32_t seen = atomicCAS(refcounts + b, old, old + d);
        if (seen == old) break;
        old = seen;
      }
    }
  }
}

inline int grid_for(int64_t work_items, int threads) {
  const DeviceInfo& di = device_info();
  int64_t blocks = (work_items + threads - 1) / threads;
  int64_t cap = int64_t(di.sm_count > 0 ? di.sm_count : 148) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return int(blocks);
}

// Grid of a grid-stride kernel capped at exactly what the SMs hold at once (from the occupancy
// calculator, looked up once per kernel): a cap above that runs the surplus CTAs as a second,
// partly filled wave.
template <typename Kernel>
inline int resident_grid_for(Kernel kernel, int64_t work_items, int threads) {
  static int per_sm = 0;
  if (per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1) n = 1;
    per_sm = n;
  }
  const DeviceInfo& di = device_info();
  int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = int64_t(di.sm_count > 0 ? di.sm_count : 148) * per_sm;
  if (blocks > cap) blocks = cap;
  return int(blocks < 1 ? 1 : blocks);
}

// Grid of a token-walking kernel: one CTA per token up to what the SMs hold at once (from the
// occupancy calculator, looked up once per kernel and CTA size).
template <typename Kernel>
inline int token_grid(Kernel kernel, int64_t num_tokens, int threads) {
  static int per_sm_cache[33] = {};  // index threads / 32; 0 = not looked up yet
  int& per_sm = per_sm_cache[threads / 32];
  if (per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1) n = 1;
    per_sm = n;
  }
  const DeviceInfo& di = device_info();
  const int64_t cap = int64_t(di.sm_count > 0 ? di.sm_count : 148) * per_sm;
  return int(num_tokens < cap ? (num_tokens < 1 ? 1 : num_tokens) : cap);
}

}  // namespace
}  // namespace kpx

using namespace kpx;

extern "C" int kpx_append(void* k_pool, void* v_pool, const kpx_kv_layout* layout,
                          const void* k_src, const void* v_src, const int64_t* slot_mapping,
                          const int32_t* pos_dev, int32_t pos_bias, int32_t num_tokens,
                          void* stream) {
  if (!layout_ok(layout) || !k_pool || !k_src || num_tokens < 0) return KPX_ERR_INVALID_ARGUMENT;
  if ((v_pool == nullptr) != (v_src == nullptr)) return KPX_ERR_INVALID_ARGUMENT;
  if (num_tokens == 0) return KPX_OK;
  if (!device_info().ok) return KPX_ERR_CUDA;
  LayoutDev L = to_dev(layout);
  int64_t work = int64_t(num_tokens) * (L.head_size * L.elt_bytes / 16) * L.num_kv_heads * (v_pool ? 2 : 1);
  const int per_tok = int(work / num_tokens);
  if (per_tok <= 1024) {
    const int threads = (per_tok + 31) / 32 * 32;
    append_token_kernel<<<token_grid(append_token_kernel, num_tokens, threads), threads, 0,
                          static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint8_t*>(k_pool), static_cast<uint8_t*>(v_pool),
        static_cast<const uint8_t*>(k_src), static_cast<const uint8_t*>(v_src), slot_mapping, pos_dev,
        pos_bias, num_tokens, L);
    return cuda_status(cudaGetLastError());
  }
  const int threads = 256;
  append_kernel<<<grid_for((work + kAppendUnroll - 1) / kAppendUnroll, threads), threads, 0,
                  static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(k_pool), static_cast<uint8_t*>(v_pool),
      static_cast<const uint8_t*>(k_src), static_cast<const uint8_t*>(v_src), slot_mapping, pos_dev,
      pos_bias, num_tokens, L);
  return cuda_status(cudaGetLastError());
}

template <typename T>
static int launch_rope(void* q, void* k, const void* v, int32_t q_heads, const int32_t* positions,
                       int32_t pos_base, const float* sin_cache, const float* cos_cache, void* k_pool, void* v_pool,
                       const LayoutDev& L, const int64_t* slot_mapping, int32_t num_tokens,
                       cudaStream_t stream, const float* q_norm_w = nullptr, const float* k_norm_w = nullptr,
                       float norm_eps = 0.f) {
  constexpr int E = Elt<T>::kPer16B;
  int groups = L.head_size / 2 / E;
  // the fused norm sums a head's squares across the `groups` consecutive lanes that hold it
  if ((q_norm_w || k_norm_w) && (groups > 32 || (groups & (groups - 1)))) return KPX_ERR_UNIMPLEMENTED;
  int64_t work = int64_t(num_tokens) *
                 (((q ? q_heads : 0) + (k ? L.num_kv_heads : 0)) * groups +
                  ((v && v_pool) ? L.num_kv_heads * L.head_size / E : 0));
  if (work == 0) return KPX_OK;
  const int threads = 256;
  rope_append_kernel<T><<<resident_grid_for(rope_append_kernel<T>, work, threads), threads, 0, stream>>>(
      static_cast<T*>(q), static_cast<T*>(k), static_cast<const T*>(v), q_heads, positions, pos_base,
      sin_cache, cos_cache, static_cast<uint8_t*>(k_pool), static_cast<uint8_t*>(v_pool),
      slot_mapping, num_tokens, L, q_norm_w, k_norm_w, norm_eps);
  return cuda_status(cudaGetLastError());
}

extern "C" int kpx_rope_append(void* q, void* k, const void* v, int32_t q_heads,
                               const int32_t* positions, int32_t pos_base, const float* sin_cache,
                               const float* cos_cache, void* k_pool, void* v_pool,
                               const kpx_kv_layout* layout, const int64_t* slot_mapping,
                               int32_t num_tokens, void* stream) {
  return kpx_norm_rope_append(q, k, v, q_heads, nullptr, nullptr, 0.f, positions, pos_base, sin_cache, cos_cache,
                              k_pool, v_pool, layout, slot_mapping, num_tokens, stream);
}

extern "C" int kpx_norm_rope_append(void* q, void* k, const void* v, int32_t q_heads, const float* q_norm_weight,
                                    const float* k_norm_weight, float norm_eps, const int32_t* positions,
                                    int32_t pos_base, const float* sin_cache, const float* cos_cache,
                                    void* k_pool, void* v_pool, const kpx_kv_layout* layout,
                                    const int64_t* slot_mapping, int32_t num_tokens, void* stream) {
  if ((q_norm_weight || k_norm_weight) && !(norm_eps >= 0.f)) return KPX_ERR_INVALID_ARGUMENT;
  if (!layout_ok(layout) || !sin_cache || !cos_cache || num_tokens < 0)
    return KPX_ERR_INVALID_ARGUMENT;
  if (q && q_heads <= 0) return KPX_ERR_INVALID_ARGUMENT;
  if (k_pool && !slot_mapping) return KPX_ERR_INVALID_ARGUMENT;
  if (k_pool && !k) return KPX_ERR_INVALID_ARGUMENT;
  if ((v_pool != nullptr) && (!v || !k_pool)) return KPX_ERR_INVALID_ARGUMENT;
  int eb = elt_bytes(layout->dtype);
  if ((layout->head_size / 2 * eb) % 16) return KPX_ERR_UNIMPLEMENTED;
  if (num_tokens == 0) return KPX_OK;
  if (!device_info().ok) return KPX_ERR_CUDA;
  LayoutDev L = to_dev(layout);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (layout->dtype) {
    case KPX_F16:
      return launch_rope<__half>(q, k, v, q_heads, positions, pos_base, sin_cache, cos_cache, k_pool, v_pool, L, slot_mapping, num_tokens, s,
                                 q_norm_weight, k_norm_weight, norm_eps);
    case KPX_BF16:
      return launch_rope<__nv_bfloat16>(q, k, v, q_heads, positions, pos_base, sin_cache, cos_cache, k_pool, v_pool, L, slot_mapping, num_tokens, s,
                                 q_norm_weight, k_norm_weight, norm_eps);
    default:
      return launch_rope<float>(q, k, v, q_heads, positions, pos_base, sin_cache, cos_cache, k_pool, v_pool, L, slot_mapping, num_tokens, s,
                                 q_norm_weight, k_norm_weight, norm_eps);
  }
}

extern "C" int kpx_sin_cos_cache(float* sin_cache, float* cos_cache, int32_t head_size,
                                 int32_t max_seq_len, float theta, void* stream) {
  if (!sin_cache || !cos_cache || head_size <= 0 || max_seq_len < 0 || !(theta > 0.f))
    return KPX_ERR_INVALID_ARGUMENT;
  if (max_seq_len == 0) return KPX_OK;
  if (!device_info().ok) return KPX_ERR_CUDA;
  const int threads = 256;
  sin_cos_kernel<<<grid_for(int64_t(head_size) * max_seq_len, threads), threads, 0,
                   static_cast<cudaStream_t>(stream)>>>(sin_cache, cos_cache, head_size,
                                                        max_seq_len, theta);
  return cuda_status(cudaGetLastError());
}

extern "C" int kpx_cow_copy_blocks(void* k_pool, void* v_pool, const kpx_kv_layout* layout,
                                   int32_t num_layers, int64_t layer_stride, const int32_t* src_ids,
                                   const int32_t* dst_ids, int32_t n, void* stream) {
  if (!layout_ok(layout) || !k_pool || !v_pool || num_layers <= 0 || n < 0 || layer_stride < 0)
    return KPX_ERR_INVALID_ARGUMENT;
  if (n == 0) return KPX_OK;
  if (!src_ids || !dst_ids) return KPX_ERR_INVALID_ARGUMENT;
  if (!device_info().ok) return KPX_ERR_CUDA;
  LayoutDev L = to_dev(layout);
  if ((layer_stride * L.elt_bytes) % 16) return KPX_ERR_INVALID_ARGUMENT;
  int64_t work = int64_t(L.head_size * L.elt_bytes / 16) * L.block_size * L.num_kv_heads * n * num_layers * 2;
  const int threads = 256;
  cow_copy_kernel<<<grid_for(work, threads), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(k_pool), static_cast<uint8_t*>(v_pool), num_layers,
      layer_stride * L.elt_bytes, src_ids, dst_ids, n, L);
  return cuda_status(cudaGetLastError());
}

extern "C" int kpx_refcount_update(int32_t* refcounts, int32_t num_blocks, const int32_t* block_ids,
                                   const int32_t* deltas, int32_t n, int32_t* error_count_dev,
                                   void* stream) {
  if (!refcounts || num_blocks <= 0 || n < 0) return KPX_ERR_INVALID_ARGUMENT;
  if (n == 0) return KPX_OK;
  if (!block_ids || !deltas) return KPX_ERR_INVALID_ARGUMENT;
  if (!device_info().ok) return KPX_ERR_CUDA;
  const int threads = 256;
  refcount_kernel<<<grid_for(n, threads), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      refcounts, num_blocks, block_ids, deltas, n, error_count_dev);
  return cuda_status(cudaGetLastError());
}
