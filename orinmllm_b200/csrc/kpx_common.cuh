// Shared device helpers for the sm_100a KV-cache kernels: mbarrier / bulk-copy
// PTX wrappers with bounded waits, element-type traits, small host utilities.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kpx.h"

namespace kpx {

// ---- host-side helpers ---------------------------------------------------------------
inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? KPX_OK : KPX_ERR_CUDA; }

#define KPX_CUDA_TRY(expr)                         \
  do {                                             \
    cudaError_t kpx_e__ = (expr);                  \
    if (kpx_e__ != cudaSuccess) return KPX_ERR_CUDA; \
  } while (0)

inline int elt_bytes(int32_t dtype) { return dtype == KPX_F32 ? 4 : 2; }

inline bool layout_ok(const kpx_kv_layout* l) {
  if (!l) return false;
  if (l->dtype != KPX_F16 && l->dtype != KPX_BF16 && l->dtype != KPX_F32) return false;
  if (l->num_kv_heads <= 0 || l->head_size <= 0 || l->block_size <= 0) return false;
  if (l->block_stride <= 0 || l->head_stride <= 0 || l->token_stride < l->head_size) return false;
  // every row must start on a 16-byte boundary (128-bit accesses, bulk copies)
  int64_t eb = elt_bytes(l->dtype);
  if ((l->block_stride * eb) % 16 || (l->head_stride * eb) % 16 || (l->token_stride * eb) % 16)
    return false;
  if ((int64_t(l->head_size) * eb) % 16) return false;
  return true;
}

// A (block, head) tile is one contiguous run of block_size*head_size elements.
inline bool tile_contiguous(const kpx_kv_layout* l) { return l->token_stride == l->head_size; }

struct DeviceInfo {
  int sm_count = 0;
  int smem_optin = 0;
  bool ok = false;
};
const DeviceInfo& device_info();  // for the current device, cached per device

// kpx_paged_decode with one more degree of freedom: batch entry b reads block-table row
// row_index[b] (device int32; nullptr = row b).  Chunked prefill uses it to run every query
// token as its own single-query attention over its sequence's row.
// With `fused` the launch is a whole decode step: seq_lens are the cached lengths (= the new
// tokens' positions), the new token's q / k rows are rotated, its k / v rows stored into the
// pools (which are written) and attended to.  `flags`: KPX_DECODE_* bits.
struct FusedStep {
  const void* k_new;
  const void* v_new;
  const float* sin_cache;
  const float* cos_cache;
};
int decode_rows(void* out, const void* q, const void* k_pool, const void* v_pool,
                const kpx_kv_layout* layout, const int32_t* block_table, int32_t max_blocks_per_seq,
                const int32_t* row_index, const int32_t* seq_lens, int32_t len_bias, int32_t batch,
                int32_t num_q_heads, float scale, void* workspace, int64_t workspace_bytes,
                void* stream, const FusedStep* fused = nullptr, int flags = 0, const void* plan = nullptr);

// ---- device-side helpers -------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false after kWaitLimit failed polls (each poll may itself
// block for a hardware-defined time slice) instead of spinning forever.
constexpr uint32_t kWaitLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = kWaitLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}

// Untiled bulk copy global -> shared through the TMA engine.  dst, src 16-byte
// aligned and bytes a multiple of 16; completion is signalled on `bar`.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- element traits: 16 bytes of T <-> floats ----
template <typename T>
struct Elt;
template <>
struct Elt<__half> {
  static constexpr int kPer16B = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
};
template <>
struct Elt<__nv_bfloat16> {
  static constexpr int kPer16B = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float x) {
    return __float2bfloat16_rn(x);
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
};
template <>
struct Elt<float> {
  static constexpr int kPer16B = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ float from_float(float x) { return x; }
  static __device__ __forceinline__ float to_float(float x) { return x; }
};

#endif  // __CUDACC__
}  // namespace kpx
