// Chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), 16-bit caches.
//
// One CTA = one tile of 128 query rows of one query head of one sequence.  Q, K, V and the
// softmax weights P live in shared memory in the 128-byte-swizzled layouts the UMMA shared
// memory descriptors describe; S = Q K^T (128x128 fp32) and the output accumulator O
// (128x128 fp32) live in tensor memory (256 columns).  Per 128-key tile:
//     tcgen05.mma  S  = Q  . K^T          (K-major A and B, 8 steps of k = 16 over d = 128)
//     threads      P  = exp2(S*c - m)     one query row per thread (TMEM lane == row),
//                                          read with tcgen05.ld, causal mask on the diagonal
//     tcgen05.mma  O += P . V             (A = P K-major, B = V MN-major as it sits in the pool)
// O is rescaled in TMEM (tcgen05.ld / st) only when a row's running maximum moved.  K/V tiles
// are gathered through the block table with cp.async into the swizzled layout (the next tile
// is in flight while the current one is being used); the pool's [16 tokens][128] tiles are
// already row-contiguous, so paging costs nothing extra.
// Every mbarrier wait is bounded and voted on by the whole CTA, so a wait that gives up ends
// the CTA in step (TMEM is freed on every path) and raises the workspace status word.
#include <vector>

#include "kpx_common.cuh"

namespace kpx {
namespace {

constexpr int kD = 128, kBS = 16, kTile = 128;
constexpr int kChunkB = kTile * 128;      // one 64-element-wide column slab: 128 rows x 128 bytes
constexpr int kOperandB = 2 * kChunkB;    // a 128 x 128 16-bit operand tile
constexpr float kLog2e = 1.4426950408889634f;

struct TileDesc {
  int32_t seq;    // row of the block table
  int32_t row0;   // first query row (global) of the tile
  int32_t nrows;  // valid rows (<= 128)
  int32_t pos0;   // cache position of row0
};

struct PrefillParams {
  void* out;
  const void* q;
  const uint8_t* k_pool;
  const uint8_t* v_pool;
  const int32_t* block_table;
  const TileDesc* tiles;
  int32_t* status;
  int64_t block_stride_b, head_stride_b;
  int64_t num_blocks;
  int32_t max_blocks_per_seq, num_q_heads, kv_mul;
  float qscale;  // softmax scale * log2(e)
};

// ---- PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)),
               "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], 128 x 128 x 16, issued by one thread
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31,%32};"
      ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte
// offsets (all >> 4), version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(const void* ptr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_u32(ptr) & 0x3FFFFu) >> 4);
  d |= uint64_t(lbo_bytes >> 4) << 16;
  d |= uint64_t(sbo_bytes >> 4) << 32;
  d |= uint64_t(1) << 46;  // descriptor version
  d |= uint64_t(2) << 61;  // SWIZZLE_128B
  return d;
}
// Instruction descriptor, kind::f16: fp32 accumulate, A/B = f16 (0) or bf16 (1), M = N = 128.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t a_format, uint32_t b_format, uint32_t b_mn_major) {
  return (1u << 4) | (a_format << 7) | (b_format << 10) | (b_mn_major << 16) | ((128u >> 3) << 17) |
         ((128u >> 4) << 24);
}

// Byte offset of (row, 16-byte chunk c16 of the 256-byte row) inside a swizzled 128x128 tile.
__device__ __forceinline__ int swz(int row, int c16) {
  return (c16 >> 3) * kChunkB + row * 128 + (((c16 & 7) ^ (row & 7)) << 4);
}

template <typename T>
struct Fmt;
template <>
struct Fmt<__half> { static constexpr uint32_t kCode = 0; };
template <>
struct Fmt<__nv_bfloat16> { static constexpr uint32_t kCode = 1; };

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T>
__device__ __forceinline__ float unpack_lo(uint32_t w);
template <typename T>
__device__ __forceinline__ float unpack_hi(uint32_t w);
template <>
__device__ __forceinline__ float unpack_lo<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w << 16); }
template <>
__device__ __forceinline__ float unpack_hi<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
template <>
__device__ __forceinline__ float unpack_lo<__half>(uint32_t w) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu)));
}
template <>
__device__ __forceinline__ float unpack_hi<__half>(uint32_t w) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
}

constexpr int kSmemBytes = 1024 /*align slack*/ + kOperandB /*Q*/ + 2 * kOperandB /*K x2*/ +
                           2 * kOperandB /*V x2*/ + 2 * kOperandB /*P_hi, P_lo*/ + 64 /*barriers, tmem slot*/ +
                           2 * kTile * 4 /*row maxima of the two column halves*/;

template <typename T>
__global__ void __launch_bounds__(256, 1) prefill_tc_kernel(const PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kOperandB;       // two buffers
  uint8_t* sV = sK + 2 * kOperandB;   // two buffers
  uint8_t* sP = sV + 2 * kOperandB;
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(sP + 2 * kOperandB);
  uint64_t* bar_o = bar_s + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o + 1);
  float* s_half = reinterpret_cast<float*>(sP + 2 * kOperandB + 64);  // [2][128] exchange between column halves

  // 8 warps: warp w and warp w+4 share TMEM lanes (= query rows) 32*(w&3)..+31; the first owns
  // columns 0..63 of S and O, the second columns 64..127.
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = tid & 127, half = tid >> 7;
  const int head = blockIdx.x % p.num_q_heads;
  const TileDesc td = p.tiles[blockIdx.x / p.num_q_heads];
  const int kvh = head / p.kv_mul;
  const int32_t* table = p.block_table + int64_t(td.seq) * p.max_blocks_per_seq;
  const int last_pos = td.pos0 + td.nrows - 1;      // newest position any row of the tile may see
  const int n_tiles = last_pos / kTile + 1;         // key tiles 0 .. n_tiles-1
  const int kv_len = last_pos + 1;

  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;
  const uint32_t lane_addr = (uint32_t((warp & 3) * 32) << 16) + uint32_t(half * 64);  // lanes and column half

  // thread t moves 16-byte chunk (t & 15) of rows (t >> 4) + 16*i, i = 0..7
  const int c16 = tid & 15, rbase = tid >> 4;
  {
    const uint8_t* qsrc = static_cast<const uint8_t*>(p.q) + (int64_t(td.row0) * p.num_q_heads + head) * (kD * 2) + c16 * 16;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = rbase + 16 * i;
      if (r < td.nrows) cp_async16(sQ + swz(r, c16), qsrc + int64_t(r) * p.num_q_heads * (kD * 2));
      else *reinterpret_cast<uint4*>(sQ + swz(r, c16)) = make_uint4(0, 0, 0, 0);
    }
  }
  auto load_kv = [&](int j, int buf) {
    uint8_t* dk = sK + buf * kOperandB;
    uint8_t* dv = sV + buf * kOperandB;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = rbase + 16 * i;         // key row inside the tile; block j*8 + i for every thread
      const int key = j * kTile + r;
      if (key < kv_len) {
        int id = __ldg(table + j * (kTile / kBS) + i);
        if (id < 0 || (p.num_blocks > 0 && id >= p.num_blocks)) {
          atomicMax(p.status, KPX_ERR_INVALID_ARGUMENT);
          id = 0;
        }
        const int64_t off = int64_t(id) * p.block_stride_b + int64_t(kvh) * p.head_stride_b + (r & 15) * (kD * 2) + c16 * 16;
        cp_async16(dk + swz(r, c16), p.k_pool + off);
        cp_async16(dv + swz(r, c16), p.v_pool + off);
      } else {  // beyond the newest token: zeros (a weight of 0 times pool garbage must stay 0)
        *reinterpret_cast<uint4*>(dk + swz(r, c16)) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(dv + swz(r, c16)) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  load_kv(0, 0);

  constexpr uint32_t kIdescQK = instr_desc(Fmt<T>::kCode, Fmt<T>::kCode, 0);
  constexpr uint32_t kIdescPV = instr_desc(Fmt<T>::kCode, Fmt<T>::kCode, 1);
  // A and B of one MMA must have the same 16-bit format (an fp16 P against a bf16 V is an
  // illegal instruction).  A single 16-bit P (2^-9 rounding for bf16, 2^-12 for fp16) costs
  // up to a few 1e-3 absolute on short sequences, beyond the 2e-3 / 1e-2 output tolerance, so
  // P is written as two 16-bit terms P = P_hi + P_lo and the output pass runs once per term.
  constexpr bool kSplitP = true;
  const int my_pos = td.pos0 + row;  // position of this thread's query row
  float m_run = -INFINITY, l_run = 0.f;
  bool failed = false;

  for (int j = 0; j < n_tiles; ++j) {
    const int buf = j & 1;
    cp_async_wait_all();
    fence_async_proxy();
    tc_fence_before();
    __syncthreads();  // tile j (and Q) visible to the tensor core; everybody is done with iteration j-1
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int o = (k >> 2) * kChunkB + (k & 3) * 32;
        umma_f16(tS, smem_desc(sQ + o, 0, 1024), smem_desc(sK + buf * kOperandB + o, 0, 1024), kIdescQK, k > 0);
      }
      umma_commit(bar_s);
    }
    if (j + 1 < n_tiles) load_kv(j + 1, buf ^ 1);  // in flight during the softmax below
    failed = !mbar_wait_bounded(bar_s, j & 1);
    if (__syncthreads_or(failed)) { failed = true; break; }
    tc_fence_after();
    // ---- softmax of this thread's row ----
    const bool diag = (j * kTile + kTile - 1) > td.pos0;  // some row of the tile is masked here
    uint32_t r[32];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      tmem_ld32(tS + lane_addr + c * 32, r);
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        float x = __uint_as_float(r[e]) * p.qscale;
        if (diag && (j * kTile + half * 64 + c * 32 + e) > my_pos) x = -INFINITY;
        mx = fmaxf(mx, x);
      }
    }
    s_half[half * kTile + row] = mx;
    __syncthreads();  // the other half of the row has published its maximum
    const float m_new = fmaxf(m_run, fmaxf(mx, s_half[(half ^ 1) * kTile + row]));
    // rows past the tile's valid rows may see nothing at all: keep them finite
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = fast_exp2(m_run - m_use);
    l_run *= alpha;
    m_run = m_new;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      tmem_ld32(tS + lane_addr + c * 32, r);
      uint32_t packed[16];
      uint32_t packed_lo[kSplitP ? 16 : 1];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float x0 = __uint_as_float(r[e]) * p.qscale, x1 = __uint_as_float(r[e + 1]) * p.qscale;
        float p0 = fast_exp2(x0 - m_use), p1 = fast_exp2(x1 - m_use);
        if (diag) {
          if ((j * kTile + half * 64 + c * 32 + e) > my_pos) p0 = 0.f;
          if ((j * kTile + half * 64 + c * 32 + e + 1) > my_pos) p1 = 0.f;
        }
        l_run += p0 + p1;
        packed[e >> 1] = pack2<T>(p0, p1);
        if (kSplitP) {
          const uint32_t hi = packed[e >> 1];
          packed_lo[e >> 1] = pack2<T>(p0 - unpack_lo<T>(hi), p1 - unpack_hi<T>(hi));
        }
      }
      // keys half*64 + c*32 .. +31 of this row = four 16-byte chunks half*8 + 4c .. +3 of the row
#pragma unroll
      for (int v = 0; v < 4; ++v)
        *reinterpret_cast<uint4*>(sP + swz(row, half * 8 + c * 4 + v)) =
            make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
      if (kSplitP) {
#pragma unroll
        for (int v = 0; v < 4; ++v)
          *reinterpret_cast<uint4*>(sP + kOperandB + swz(row, half * 8 + c * 4 + v)) =
              make_uint4(packed_lo[4 * v], packed_lo[4 * v + 1], packed_lo[4 * v + 2], packed_lo[4 * v + 3]);
      }
    }
    // ---- rescale O where a running maximum moved (the previous O += P V has completed) ----
    if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tmem_ld32(tO + lane_addr + c * 32, r);
#pragma unroll
        for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
        tmem_st32(tO + lane_addr + c * 32, r);
      }
    }
    fence_async_proxy();
    tc_fence_before();
    __syncthreads();  // P complete, S fully read, O rescaled
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        // A = P: keys 16k.. of every row (K-major); B = V: key rows 16k.. , d along MN
        const uint64_t a = smem_desc(sP + (k >> 2) * kChunkB + (k & 3) * 32, 0, 1024);
        const uint64_t b = smem_desc(sV + buf * kOperandB + k * (16 * 128), kChunkB, 1024);
        umma_f16(tO, a, b, kIdescPV, (j > 0 || k > 0) ? 1u : 0u);
      }
      if (kSplitP) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t a = smem_desc(sP + kOperandB + (k >> 2) * kChunkB + (k & 3) * 32, 0, 1024);
          const uint64_t b = smem_desc(sV + buf * kOperandB + k * (16 * 128), kChunkB, 1024);
          umma_f16(tO, a, b, kIdescPV, 1u);
        }
      }
      umma_commit(bar_o);
    }
    failed = !mbar_wait_bounded(bar_o, j & 1);
    if (__syncthreads_or(failed)) { failed = true; break; }
    tc_fence_after();
  }

  if (!failed) {
    // ---- epilogue: out = O / l ----
    // the row sum is the sum of the two column halves
    s_half[half * kTile + row] = l_run;
    __syncthreads();
    const float l_row = l_run + s_half[(half ^ 1) * kTile + row];
    const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
    uint8_t* orow = static_cast<uint8_t*>(p.out) + (int64_t(td.row0 + row) * p.num_q_heads + head) * (kD * 2) +
                    half * 128;
    uint32_t r[32];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      tmem_ld32(tO + lane_addr + c * 32, r);
      if (row < td.nrows) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 w;
          w.x = pack2<T>(__uint_as_float(r[8 * v + 0]) * inv, __uint_as_float(r[8 * v + 1]) * inv);
          w.y = pack2<T>(__uint_as_float(r[8 * v + 2]) * inv, __uint_as_float(r[8 * v + 3]) * inv);
          w.z = pack2<T>(__uint_as_float(r[8 * v + 4]) * inv, __uint_as_float(r[8 * v + 5]) * inv);
          w.w = pack2<T>(__uint_as_float(r[8 * v + 6]) * inv, __uint_as_float(r[8 * v + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + (c * 4 + v) * 16) = w;
        }
      }
    }
  } else if (tid == 0) {
    atomicMax(p.status, KPX_ERR_DEVICE_TIMEOUT);
  }
  cp_async_wait_all();  // nothing of ours may still be landing in shared memory
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace

// Host side: tile list -> workspace, launch.  Returns KPX_ERR_UNIMPLEMENTED when the layout
// or dtype is outside this path so that the caller can fall back to the streaming path.
int prefill_tc(void* out, const void* q, const void* k_pool, const void* v_pool, const kpx_kv_layout* layout,
               const int32_t* block_table, int32_t max_blocks_per_seq, const int32_t* cu_q_lens_host,
               const int32_t* start_pos_host, int32_t batch, int32_t num_q_heads, float scale, void* tile_area,
               int64_t tile_area_bytes, int32_t* status, cudaStream_t stream) {
  if (layout->dtype == KPX_F32 || layout->head_size != kD || layout->block_size != kBS || !tile_contiguous(layout) ||
      !block_table)
    return KPX_ERR_UNIMPLEMENTED;
  std::vector<TileDesc> tiles;
  for (int32_t b = 0; b < batch; ++b) {
    const int32_t n = cu_q_lens_host[b + 1] - cu_q_lens_host[b];
    for (int32_t t0 = 0; t0 < n; t0 += kTile)
      tiles.push_back(TileDesc{b, cu_q_lens_host[b] + t0, n - t0 < kTile ? n - t0 : kTile, start_pos_host[b] + t0});
  }
  if (tiles.empty()) return KPX_OK;
  if (int64_t(tiles.size() * sizeof(TileDesc)) > tile_area_bytes) return KPX_ERR_WORKSPACE_TOO_SMALL;
  KPX_CUDA_TRY(cudaMemcpyAsync(tile_area, tiles.data(), tiles.size() * sizeof(TileDesc), cudaMemcpyHostToDevice, stream));
  PrefillParams p;
  p.out = out;
  p.q = q;
  p.k_pool = static_cast<const uint8_t*>(k_pool);
  p.v_pool = static_cast<const uint8_t*>(v_pool);
  p.block_table = block_table;
  p.tiles = static_cast<const TileDesc*>(tile_area);
  p.status = status;
  p.block_stride_b = layout->block_stride * 2;
  p.head_stride_b = layout->head_stride * 2;
  p.num_blocks = layout->num_blocks;
  p.max_blocks_per_seq = max_blocks_per_seq;
  p.num_q_heads = num_q_heads;
  p.kv_mul = num_q_heads / layout->num_kv_heads;
  p.qscale = scale * kLog2e;
  const unsigned grid = unsigned(tiles.size()) * unsigned(num_q_heads);
  if (layout->dtype == KPX_F16) {
    static int done = -1;
    int dev = 0;
    KPX_CUDA_TRY(cudaGetDevice(&dev));
    if (done != dev) {
      KPX_CUDA_TRY(cudaFuncSetAttribute(prefill_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      done = dev;
    }
    prefill_tc_kernel<__half><<<grid, 256, kSmemBytes, stream>>>(p);
  } else {
    static int done = -1;
    int dev = 0;
    KPX_CUDA_TRY(cudaGetDevice(&dev));
    if (done != dev) {
      KPX_CUDA_TRY(cudaFuncSetAttribute(prefill_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      done = dev;
    }
    prefill_tc_kernel<__nv_bfloat16><<<grid, 256, kSmemBytes, stream>>>(p);
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace kpx
