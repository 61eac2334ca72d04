// Chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), 16-bit caches.
//
// One CTA = two items (128 query rows x one query head each) of one sequence that share a KV
// head, so one stream of K/V tiles serves both.  576 threads in roles:
//   warp 17      TMA: Q boxes, then per 128-key tile the (block, head) boxes of K and V through
//                the block table into 128-byte-swizzled shared memory (two stages each); it also
//                waits for the tiles to land and publishes the count in a progress word
//   warp 16      walks the MMA schedule in step, one elected lane issues tcgen05.mma:
//                S_x = Q_x K^T  into tensor memory (128 columns per item) and  O_x += P_x V
//                (A = P read from tensor memory, B = V MN-major as it sits in the pool);
//                completion is committed to mbarriers.  In its loop it polls no barrier: one
//                plain load of the progress words shows what a step needs
//   warps 0..7   softmax of item 0, warps 8..15 softmax of item 1: S_x -> P_x = exp2(S*c - m)
//                written over S_x as two 16-bit terms (tcgen05.ld / st; two threads per query
//                row), causal mask on the diagonal, running maximum moved lazily, O_x rescaled
//                in tensor memory when it moves; P is handed over in two waves per tile (each
//                warp counts them in its progress word)
// The MMA order  PV_0(j) QK_0(j+1) | PV_1(j) QK_1(j+1)  keeps the tensor core on one item while
// the softmax threads work on the other.
// A CTA may own only a range of its pair's key tiles (a call with too few pairs to fill the SMs
// is cut that way): it then leaves unnormalised rows with their maximum and sum in a slot of the
// work area, and prefill_merge_kernel combines the parts.
// Every mbarrier wait is bounded; a role that gives up raises a CTA-wide flag that ends the
// other roles' waits, TMEM is freed on every path and the workspace status word is raised.
#include <cuda.h>  // CUtensorMap and the enums of cuTensorMapEncodeTiled (types only; no libcuda link)

#include <algorithm>
#include <atomic>
#include <type_traits>
#include <vector>

#include "kpx_common.cuh"

namespace kpx {
namespace {

constexpr int kD = 128, kBS = 16, kTile = 128;
constexpr int kChunkB = kTile * 128;      // one 64-element-wide column slab: 128 rows x 128 bytes
constexpr int kOperandB = 2 * kChunkB;    // a 128 x 128 16-bit operand tile
constexpr float kLog2e = 1.4426950408889634f;

// One unit of work: 128 query rows of one query head.
struct ItemDesc {
  int32_t row0;   // first query row (global) of the tile
  int32_t nrows;  // valid rows (<= 128); 0 = no item
  int32_t pos0;   // cache position of row0
  int32_t head;   // query head
};
// One CTA: two items of one sequence that share a KV head, so that one stream of K/V tiles
// serves both.  it[1] is always present and sees at least as many keys as it[0].
struct PairDesc {
  int32_t seq;  // row of the block table
  int32_t kvh;
  ItemDesc it[2];
  // This CTA's share of the pair's key tiles [tile0, tile1) and, when the pair is cut into
  // several such shares, the slot its unnormalised result goes to (-1: the CTA owns the whole
  // pair and writes the output rows itself).
  int32_t tile0, tile1, part, pad;
};
// One item whose key range was cut: `parts` slots to merge into its output rows.
struct MergeDesc {
  ItemDesc it;
  int32_t slot[4];
  int32_t parts, x;  // x: which item of its pair (position inside the slot)
  int32_t pad[2];
};
// A slot holds, for both items of a pair, 128 rows of [O (128 floats), m, l].
constexpr int kPartRow = kD + 2;
constexpr int64_t kPartItemFloats = int64_t(kTile) * kPartRow;
constexpr int64_t kPartSlotFloats = 2 * kPartItemFloats;
constexpr int kMaxPartSlots = 320;  // two per SM of the largest device planned for
inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

struct PrefillParams {
  void* out;
  const int32_t* block_table;
  const PairDesc* pairs;
  float* partials;  // slots of kPartSlotFloats floats
  int32_t* status;
  int64_t num_blocks;
  int32_t max_blocks_per_seq, num_q_heads, kv_mul;
  float qscale;  // softmax scale * log2(e)
  // Polls a bounded wait makes before it gives up (kWaitLimit), and, for the test of that path
  // only, the CTA one of whose tiles is announced to its barrier but never requested (-1: none;
  // the tile is chosen by the bits above the low 16, see the loader).
  uint32_t wait_limit;
  int32_t withhold_cta;
};

// ---- PTX wrappers -----------------------------------------------------------------------
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
// D[tmem] (+)= A[tmem] * B[smem]: A is read from tensor memory (row = lane, two 16-bit k values
// per 32-bit column, 8 columns per k = 16 step)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
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


// Tensor memory is allocated per CTA and the occupancy calculator places one CTA of this kernel
// per SM whatever its shared-memory and register footprint, so the overlap of softmax and
// tensor-core work has to happen inside the CTA: each CTA carries two items (A, B) and
// alternates between them.
constexpr int kKTilesWord = 16, kVTilesWord = 17, kAbortWord = 18;  // progress words, see the kernel
constexpr int kMmaWarp = 16, kLoadWarp = 17;  // warps 0..7: softmax of item 0, warps 8..15: of item 1
constexpr int kThreads = 576;
constexpr int kSmemBytes = 1024 /*align slack*/ + 2 * kOperandB /*Q of A, B*/ + 2 * kOperandB /*K x2*/ +
                           2 * kOperandB /*V x2*/ + 256 /*barriers, tmem slot, abort flag*/ +
                           2 * 2 * kTile * 4 /*per item: exchange between the two column halves of a row*/;

// Barrier among the 256 softmax threads of one item (hardware barrier `id` = 1 or 2; barrier 0
// is __syncthreads).
__device__ __forceinline__ void softmax_sync(int id) { asm volatile("bar.sync %0, 256;" ::"r"(id) : "memory"); }
// The same with a vote: true when any of the 256 threads passes true.
__device__ __forceinline__ bool softmax_sync_or(int id, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %2, 0;\n\t"
      "bar.red.or.pred q, %1, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"(id), "r"(uint32_t(pred))
      : "memory");
  return out != 0;
}
// Bounded wait that also gives up as soon as another role of the CTA has given up.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) {
      __nanosleep(64);
      if ((i & 127) == 0 && *abort_flag) return false;
    }
  }
  *abort_flag = 1;
  return false;
}
// Tiled TMA loads, each into this CTA's own shared memory: a box of the tensor map lands there,
// 128-byte swizzled, and its bytes are counted on the mbarrier.
__device__ __forceinline__ void tma_load_3d(void* dst, const void* tmap, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst)), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const void* tmap, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], "
      "[%6];"
      ::"r"(smem_u32(dst)), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t addr, uint32_t* r) {
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
}
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Largest of 32 scores; with kMasked, scores of keys e > limit (newer than the query) do not count.
template <bool kMasked>
__device__ __forceinline__ float max32(const uint32_t* r, int limit, float mx) {
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    float a = __uint_as_float(r[e]), b = __uint_as_float(r[e + 1]);
    if (kMasked) {
      if (e > limit) a = -INFINITY;
      if (e + 1 > limit) b = -INFINITY;
    }
    mx = fmaxf(mx, fmaxf(a, b));
  }
  return mx;
}

__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(addr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t addr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// How many 16-bit terms carry a weight p into the P V product.  One term was measured for both
// formats and fails the output tolerance on short sequences: bf16 (2^-9 relative rounding) by a
// few 1e-3 absolute, fp16 (2^-11) within 2e-3 absolute but up to 2.5e-2 relative on outputs near
// zero (a 37-token sequence, where a few weights carry the row and their rounding errors do not
// average out), against a bound of 1e-2.  Both formats therefore carry p = P_hi + P_lo and run
// P V twice; the single-term form stays behind this constant (it is 12 % faster: 224 against
// 250 us per layer on 4 x 2048 tokens) for a caller whose tolerance allows it.
template <typename T>
struct PTerms { static constexpr int kCount = 2; };

// P reaches the MMA warp in kWaves hand-overs per 128-key tile: a thread's 64 keys are four
// groups of 16 (one k = 16 step of the P V product each); after every 4 / kWaves groups the warp
// announces them, and the MMA warp issues the P V steps of that wave while the softmax threads
// are still at the exponentials of the next one.
constexpr int kWaves = 2;
constexpr int kGroupsPerWave = 4 / kWaves;

// Weights of 16 keys, group h (0 or 1) of a 32-column slice of S whose scores are in r[0..31]:
// p = exp2(s * qscale - m), written over the slice as P_hi (columns 8h..8h+7, two keys each) and,
// with two terms, P_lo = p - P_hi (columns 16+8h..); lsum += p.  Keys e > limit are masked.
template <typename T, bool kMasked>
__device__ __forceinline__ void weights16(uint32_t taddr, int h, const uint32_t* r, float qscale, float neg_m,
                                          int limit, float2& lsum) {
  const float2 sc = make_float2(qscale, qscale), nm = make_float2(neg_m, neg_m), m1 = make_float2(-1.f, -1.f);
  uint32_t hi[8], lo[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = h * 16 + 2 * i;
    const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), sc, nm);
    float2 w = make_float2(fast_exp2(x.x), fast_exp2(x.y));
    if (kMasked) {
      if (e > limit) w.x = 0.f;
      if (e + 1 > limit) w.y = 0.f;
    }
    lsum = __fadd2_rn(lsum, w);
    const uint32_t hw = pack2<T>(w.x, w.y);
    hi[i] = hw;
    if (PTerms<T>::kCount == 2) {
      const float2 d = __ffma2_rn(make_float2(unpack_lo<T>(hw), unpack_hi<T>(hw)), m1, w);
      lo[i] = pack2<T>(d.x, d.y);
    }
  }
  tmem_st8(taddr + h * 8, hi);
  if (PTerms<T>::kCount == 2) tmem_st8(taddr + 16 + h * 8, lo);
}

// Per-thread softmax state of one item: this thread owns (row, column half) of S and O.
struct RowState {
  float m = -INFINITY;            // running maximum (scaled scores), moved lazily
  float2 l = {0.f, 0.f};          // running sum of weights, as an even/odd pair
};

// A running maximum is only moved when the tile's maximum exceeds it by more than this (in
// log2 units): weights stay below 2^8, and O is rescaled in far fewer tiles.
constexpr float kLazyMax = 8.f;

// Softmax of key tile j of one item: S (tensor memory, 128 columns at tS) -> P over S, handed to
// the MMA warp wave by wave (this warp's progress word counts the waves it has announced); O
// (which holds something when has_o) is rescaled first where the row maximum moved.  Called by
// the 256 softmax threads of the item (contains their barrier `bar_id`, which also carries the
// vote on `bad`: a thread whose wait for S ran out).  Returns false, in all 256 threads alike,
// when any of them passed bad.
template <typename T>
__device__ __forceinline__ bool softmax_tile(uint32_t tS, uint32_t tO, uint32_t lane_addr, int row, int half,
                                             float qscale, int j, bool has_o, int pos0, float* s_half,
                                             int bar_id, RowState& st, bool bad, volatile uint32_t* my_word,
                                             uint32_t waves_before, int lane) {
  const int my_pos = pos0 + row;
  const bool diag = (j * kTile + kTile - 1) > pos0;  // some row of this item is masked in this tile
  const int limit0 = my_pos - (j * kTile + half * 64);   // keys e > limit are newer than the query
  uint32_t r0[32], r1[32];
  tmem_ld32_nowait(tS + lane_addr, r0);
  tmem_ld32_nowait(tS + lane_addr + 32, r1);
  tmem_wait_ld();
  float mx;
  if (diag) mx = max32<true>(r1, limit0 - 32, max32<true>(r0, limit0, -INFINITY));
  else mx = max32<false>(r1, 0, max32<false>(r0, 0, -INFINITY));
  s_half[half * kTile + row] = mx;
  if (softmax_sync_or(bar_id, bad)) return false;  // the other half of the row has published its maximum
  const float m_tile = fmaxf(mx, s_half[(half ^ 1) * kTile + row]) * qscale;
  float alpha = 1.f;
  if (m_tile > st.m + kLazyMax || st.m == -INFINITY) {  // (-inf + 8 is -inf: the first tile always moves it)
    const float m_new = (m_tile == -INFINITY) ? 0.f : m_tile;
    alpha = fast_exp2(st.m - m_new);
    st.m = m_new;
    st.l.x *= alpha;
    st.l.y *= alpha;
  }
  // O += P V of the previous tile has completed (the MMA that produced S was issued after it), and
  // none of this tile's is issued before every warp of the item has announced its first wave
  if (has_o && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
    for (int c = 0; c < 8; ++c) {
      uint32_t o[8];
      tmem_ld8(tO + lane_addr + c * 8, o);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
      tmem_st8(tO + lane_addr + c * 8, o);
    }
  }
  const float neg_m = -st.m;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint32_t* r = g < 2 ? r0 : r1;
    const uint32_t taddr = tS + lane_addr + (g >> 1) * 32;
    const int limit = limit0 - (g >> 1) * 32;
    if (diag) weights16<T, true>(taddr, g & 1, r, qscale, neg_m, limit, st.l);
    else weights16<T, false>(taddr, g & 1, r, qscale, neg_m, limit, st.l);
    if ((g + 1) % kGroupsPerWave == 0) {
      tmem_wait_st();  // this warp's part of the wave (and a rescaled O) is in tensor memory
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        *my_word = waves_before + uint32_t(g / kGroupsPerWave) + 1u;
      }
    }
  }
  return true;
}

// out rows of one item = O / l.  Called by the 256 softmax threads of the item (contains their
// barrier).  A thread holds 128 contiguous bytes of one row, so a warp's direct stores would hit
// 32 different rows; the rows go through `stage` (32 KB of shared memory nobody else touches any
// more: the item's Q tile) and leave as whole 256-byte rows, 16 lanes each.
template <typename T>
__device__ __forceinline__ void write_item(uint32_t tO, uint32_t lane_addr, int row, int half, const ItemDesc& it,
                                           int num_q_heads, void* out, float* s_half, int bar_id, const RowState& st,
                                           uint8_t* stage) {
  const float l_mine = st.l.x + st.l.y;
  softmax_sync(bar_id);  // earlier readers of the exchange area are done
  s_half[half * kTile + row] = l_mine;
  softmax_sync(bar_id);
  const float l_row = l_mine + s_half[(half ^ 1) * kTile + row];
  const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
  uint32_t r[32];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    tmem_ld32(tO + lane_addr + c * 32, r);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint4 w;
      w.x = pack2<T>(__uint_as_float(r[8 * v + 0]) * inv, __uint_as_float(r[8 * v + 1]) * inv);
      w.y = pack2<T>(__uint_as_float(r[8 * v + 2]) * inv, __uint_as_float(r[8 * v + 3]) * inv);
      w.z = pack2<T>(__uint_as_float(r[8 * v + 4]) * inv, __uint_as_float(r[8 * v + 5]) * inv);
      w.w = pack2<T>(__uint_as_float(r[8 * v + 6]) * inv, __uint_as_float(r[8 * v + 7]) * inv);
      // 16-byte chunk (half*8 + c*4 + v) of the row, stored at a position rotated by the row so
      // that the 32 rows of a warp spread over the banks
      const int chunk = half * 8 + c * 4 + v;
      *reinterpret_cast<uint4*>(stage + row * 256 + ((chunk ^ (row & 15)) << 4)) = w;
    }
  }
  softmax_sync(bar_id);  // the whole tile is staged
  const int t = half * kTile + row;  // 0..255 within the item's threads
  const int chunk = t & 15;
  uint8_t* obase = static_cast<uint8_t*>(out) + (int64_t(it.row0) * num_q_heads + it.head) * (kD * 2) + chunk * 16;
#pragma unroll
  for (int i = 0; i < kTile / 16; ++i) {
    const int rr = (t >> 4) + 16 * i;
    if (rr < it.nrows)
      *reinterpret_cast<uint4*>(obase + int64_t(rr) * num_q_heads * (kD * 2)) =
          *reinterpret_cast<const uint4*>(stage + rr * 256 + ((chunk ^ (rr & 15)) << 4));
  }
}

// The same rows, unnormalised, for a CTA that saw only part of the keys: [O (128), m, l] per row
// into its slot; the merge kernel combines the parts.
__device__ __forceinline__ void write_partial(uint32_t tO, uint32_t lane_addr, int row, int half, float* dst,
                                              float* s_half, int bar_id, const RowState& st) {
  const float l_mine = st.l.x + st.l.y;
  softmax_sync(bar_id);  // earlier readers of the exchange area are done
  s_half[half * kTile + row] = l_mine;
  softmax_sync(bar_id);
  float* drow = dst + int64_t(row) * kPartRow;
  if (half == 0) {
    drow[kD] = st.m;
    drow[kD + 1] = l_mine + s_half[kTile + row];
  }
  uint32_t r[32];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    tmem_ld32(tO + lane_addr + c * 32, r);
#pragma unroll
    for (int v = 0; v < 16; ++v)  // rows are 130 floats long: 8-byte alignment only
      *reinterpret_cast<uint2*>(drow + half * 64 + c * 32 + 2 * v) = make_uint2(r[2 * v], r[2 * v + 1]);
  }
}

// Output rows of an item whose keys were cut into parts: out = sum_p 2^(m_p - M) O_p / sum_p 2^(m_p - M) l_p.
// blockIdx.x = item, blockIdx.y = group of 16 rows; threadIdx.x = d, threadIdx.y takes every 4th row.
constexpr int kMergeRowsPerCta = 16, kMergeRowLanes = 4;
template <typename T>
__global__ void __launch_bounds__(kD* kMergeRowLanes)
    prefill_merge_kernel(T* __restrict__ out, const float* __restrict__ partials, const MergeDesc* __restrict__ descs,
                         int num_q_heads) {
  const MergeDesc md = descs[blockIdx.x];
  const int d = threadIdx.x;
#pragma unroll
  for (int i = 0; i < kMergeRowsPerCta / kMergeRowLanes; ++i) {
    const int row = blockIdx.y * kMergeRowsPerCta + i * kMergeRowLanes + threadIdx.y;
    if (row >= md.it.nrows) continue;
    // every part's (m, l) first, then the weights, then the O values: two rounds of independent
    // loads.  A part in which the row saw no key (l = 0) carries a placeholder maximum and does
    // not count.
    const float* base = partials + md.x * kPartItemFloats + int64_t(row) * kPartRow;
    float mp[4], lp[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const bool on = p < md.parts;
      const float* prow = base + (on ? md.slot[p] : md.slot[0]) * kPartSlotFloats;
      mp[p] = prow[kD];
      lp[p] = on ? prow[kD + 1] : 0.f;
    }
    float M = -INFINITY;
#pragma unroll
    for (int p = 0; p < 4; ++p)
      if (lp[p] > 0.f) M = fmaxf(M, mp[p]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float w = lp[p] > 0.f ? fast_exp2(mp[p] - M) : 0.f;
      const float* prow = base + (p < md.parts ? md.slot[p] : md.slot[0]) * kPartSlotFloats;
      const float o = prow[d];
      acc = lp[p] > 0.f ? fmaf(o, w, acc) : acc;  // (a skipped part may hold anything, NaN included)
      L = fmaf(lp[p], w, L);
    }
    out[(int64_t(md.it.row0 + row) * num_q_heads + md.it.head) * kD + d] = Elt<T>::from_float(L > 0.f ? acc / L : 0.f);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
    prefill_tc_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap map_q,
                      const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                  // Q of item 0, Q of item 1
  uint8_t* sK = sQ + 2 * kOperandB;    // two stages
  uint8_t* sV = sK + 2 * kOperandB;    // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * kOperandB);
  uint64_t* q_full = bars;         // Q of both items has landed
  uint64_t* k_full = bars + 1;     // [2] stage holds K(j)
  uint64_t* v_full = bars + 3;     // [2] stage holds V(j)
  uint64_t* k_free = bars + 5;     // [2] every MMA reading the stage has completed
  uint64_t* v_free = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;     // [2] S of item x complete (and every earlier MMA)
  uint64_t* o_full = bars + 11;    // [2] last O += P V of item x complete
  constexpr int kNumBars = 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  // Progress words the MMA warp reads with one plain load (lane i reads word i, see there):
  // [0..7] / [8..15] waves of P announced by the softmax warps of item 0 / 1, [16] K tiles and
  // [17] V tiles that have landed, [18] the CTA's give-up flag.
  volatile uint32_t* flags = reinterpret_cast<volatile uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(flags + kAbortWord);
  float* s_half = reinterpret_cast<float*>(sV + 2 * kOperandB + 256);  // [2 items][2][128]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const PairDesc pd = p.pairs[blockIdx.x];
  const int last_pos = pd.it[1].pos0 + pd.it[1].nrows - 1;  // newest position any row of the pair may see
  const int kv_len = last_pos + 1;
  const int tilesB = last_pos / kTile + 1;                   // key tiles 0 .. tilesB-1 of item 1
  const int tilesA = pd.it[0].nrows > 0 ? (pd.it[0].pos0 + pd.it[0].nrows - 1) / kTile + 1 : 0;  // <= tilesB
  // this CTA walks the key tiles j0 + j, j = 0 .. nB-1 (item 0: .. nA-1)
  const int j0 = pd.tile0;
  const int nB = min(tilesB, pd.tile1) - j0;
  const int nA = max(0, min(tilesA, pd.tile1) - j0);
  const bool ragged = (kv_len % kTile) != 0;                 // the last tile has rows past the newest token

  if (tid == 0) {
    for (int i = 0; i < kNumBars; ++i) mbar_init(bars + i, 1u);
    for (int i = 0; i < 32; ++i) flags[i] = 0;
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;  // columns: S of item 0, S of item 1, O of item 0, O of item 1

  if (warp == kLoadWarp) {
    // ===== loader: TMA boxes of Q, then of K(j), V(j) through the block table =====
    const int32_t* table = p.block_table + int64_t(pd.seq) * p.max_blocks_per_seq;
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, (nA > 0 ? 2u : 1u) * kOperandB);
#pragma unroll
      for (int x = 0; x < 2; ++x)
        if ((x ? nB : nA) > 0) {
          tma_load_3d(sQ + x * kOperandB, &map_q, 0, pd.it[x].head, pd.it[x].row0, q_full);
          tma_load_3d(sQ + x * kOperandB + kChunkB, &map_q, 64, pd.it[x].head, pd.it[x].row0, q_full);
        }
    }
    bool ok = true;
    for (int j = 0; j < nB && ok; ++j) {
      const int stage = j & 1, use = j >> 1;
      const int left = kv_len - (j0 + j) * kTile;                 // tokens from the start of this tile
      const int nblk = left >= kTile ? kTile / kBS : (left + kBS - 1) / kBS;
      // lanes 0..15: block (lane >> 1), 64-element slab (lane & 1)
      int id = 0;
      if (lane < 2 * nblk) {
        id = __ldg(table + (j0 + j) * (kTile / kBS) + (lane >> 1));
        if (id < 0 || (p.num_blocks > 0 && id >= p.num_blocks)) {
          atomicMax(p.status, KPX_ERR_INVALID_ARGUMENT);
          id = 0;
        }
      }
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        uint64_t* full = (kv ? v_full : k_full) + stage;
        uint64_t* free_bar = (kv ? v_free : k_free) + stage;
        if (use > 0) ok = ok && wait_or_abort(free_bar, uint32_t((use - 1) & 1), abort_flag, p.wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) mbar_arrive_expect_tx(full, uint32_t(nblk) * (kBS * kD * 2));
        __syncwarp();
        // test knob: CTA (withhold_cta & 0xffff) never requests one tile it has announced:
        // (withhold_cta >> 16) = 0: K of tile 0, 1: V of tile 0, 2: K of tile 1
        const int what = p.withhold_cta >> 16;
        const bool withheld = p.withhold_cta >= 0 && int(blockIdx.x) == (p.withhold_cta & 0xffff) &&
                              j == (what == 2 ? 1 : 0) && kv == (what == 1 ? 1 : 0);
        if (lane < 2 * nblk && !withheld) {
          uint8_t* dst = (kv ? sV : sK) + stage * kOperandB + (lane & 1) * kChunkB + (lane >> 1) * (kBS * 128);
          tma_load_4d(dst, kv ? &map_v : &map_k, (lane & 1) * 64, 0, pd.kvh, id, full);
        }
      }
      // Tell the MMA warp what has landed: it reads all it needs for a step with one load of
      // the progress words instead of polling these barriers one after the other.
      if (ok) ok = wait_or_abort(k_full + stage, uint32_t(use & 1), abort_flag, p.wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (ok && lane == 0) {
        __threadfence_block();
        flags[kKTilesWord] = uint32_t(j + 1);
      }
      if (ok) ok = wait_or_abort(v_full + stage, uint32_t(use & 1), abort_flag, p.wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (ok && ragged && j0 + j == tilesB - 1) {
        // V rows past the newest token must be zero (a weight of 0 times pool garbage must stay
        // 0); the boxes have landed, the last one covers some of these rows
        uint8_t* v = sV + stage * kOperandB;
        for (int i = left * 16 + lane; i < kTile * 16; i += 32) {  // 16-byte pieces of rows left..127
          const int r = i >> 4, c = i & 15;
          *reinterpret_cast<uint4*>(v + (c >> 3) * kChunkB + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_async_proxy();
      }
      __syncwarp();
      if (ok && lane == 0) {
        __threadfence_block();
        flags[kVTilesWord] = uint32_t(j + 1);
      }
    }
  } else if (warp == kMmaWarp) {
    // ===== MMA issue.  The whole warp walks the schedule in step (every wait result is made
    // warp-uniform) and one elected lane issues, so that descriptors and addresses stay in
    // uniform registers =====
    constexpr uint32_t kIdescQK = instr_desc(Fmt<T>::kCode, Fmt<T>::kCode, 0);
    constexpr uint32_t kIdescPV = instr_desc(Fmt<T>::kCode, Fmt<T>::kCode, 1);
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    // descriptors of the operand bases; the k steps add to the 16-byte-unit address field
    const uint64_t dq0 = smem_desc(sQ, 0, 1024), dk0 = smem_desc(sK, 0, 1024), dv0 = smem_desc(sV, kChunkB, 1024);
    constexpr uint64_t kNextOperand = uint64_t(kOperandB >> 4);  // second item's Q, second stage of K / V
    bool ok = true;
    // S_x = Q_x K(j)^T: 8 steps of k = 16 over d = 128 (4 steps per 64-element slab)
    auto issue_qk = [&](int x, int j) {
      const uint64_t a = dq0 + uint64_t(x) * kNextOperand, b = dk0 + uint64_t(j & 1) * kNextOperand;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const uint64_t o = uint64_t(((s >> 2) * kChunkB + (s & 3) * 32) >> 4);
        umma_f16(tm + x * 128, a + o, b + o, kIdescQK, s > 0);
      }
      umma_commit(s_full + x);
    };
    // Wave w of O_x += P_hi V(j) (+ P_lo V(j) where P has two terms, see PTerms).  A = P from
    // tensor memory: keys 16s.. of every row sit in 8 columns; B = V: key rows 16s.., d along MN.
    // A and B of one MMA must have the same 16-bit format (an fp16 P against a bf16 V is an
    // illegal instruction).  The two threads of a query row own keys 0..63 and 64..127 and work
    // through them in step, so a wave is the k steps g and g + 4 for its groups g.
    auto issue_pv_wave = [&](int x, int j, int w) {
      const uint32_t tP = tm + x * 128, tO = tm + 256 + x * 128;
      const uint64_t b = dv0 + uint64_t(j & 1) * kNextOperand;
#pragma unroll
      for (int gg = 0; gg < kGroupsPerWave; ++gg) {
        const int g = w * kGroupsPerWave + gg;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int s = g + 4 * hh;
          const uint32_t a = tP + (s >> 1) * 32 + (s & 1) * 8;
          const uint64_t bs = b + uint64_t((s * 16 * 128) >> 4);
          umma_f16_ts(tO, a, bs, kIdescPV, (j > 0 || g > 0 || hh > 0) ? 1u : 0u);
          if (PTerms<T>::kCount == 2) umma_f16_ts(tO, a + 16, bs, kIdescPV, 1u);
        }
      }
    };
    auto wait = [&](uint64_t* bar, int parity) {
      ok = ok && __all_sync(0xffffffffu, wait_or_abort(bar, uint32_t(parity), abort_flag, p.wait_limit));
      tc_fence_after();
      return ok;
    };
    if (wait(q_full, 0) && wait(k_full, 0)) {
      if (elect_one()) {
        if (nA > 0) issue_qk(0, 0);
        issue_qk(1, 0);
        umma_commit(k_free);
      }
      __syncwarp();
    }
    // This warp is one dependent instruction stream next to sixteen busy softmax warps, and what
    // it does between two batches of MMAs is time the tensor pipe stands still.  A per-step
    // timeline showed every look at shared memory after a batch, a barrier poll or a plain load,
    // to take it 200 - 350 clocks, complete or not, and a step needs up to four barriers.  So it
    // polls no barrier in the loop: the softmax warps and the loader publish their progress in
    // plain words, and ONE load, lane i reading word i, shows everything a step needs: the
    // item's eight softmax warps (lanes 0..7), the K and V tiles landed (lanes 8, 9), the
    // give-up flag (lane 10).  The steps are unrolled with item and wave as constants.
    const int word_other = lane < 8 ? 0 : lane < 11 ? lane + 8 : 19;  // lanes 8..10 read words 16..18, the rest a word that stays 0
    auto step = [&](auto item, auto wave, int j) -> bool {
      constexpr int x = decltype(item)::value, w = decltype(wave)::value;
      const int n_x = x ? nB : nA;
      const bool scores_next = w + 1 == kWaves && j + 1 < n_x;
      uint32_t need = 0;
      if (lane < 8) need = uint32_t(j * kWaves + w + 1);
      else if (lane == 8) need = scores_next ? uint32_t(j + 2) : 0u;
      else if (lane == 9) need = uint32_t(j + 1);
      const volatile uint32_t* word = flags + (lane < 8 ? x * 8 + lane : word_other);
      bool ready = false;
      for (uint32_t i = 0; i < p.wait_limit; ++i) {
        const uint32_t v = *word;
        const uint32_t good = __ballot_sync(0xffffffffu, lane == 10 ? v == 0 : v >= need);
        if (good == 0xffffffffu) {
          ready = true;
          break;
        }
        if (!((good >> 10) & 1u)) return false;  // another role has given up
      }
      if (!ready) {
        *abort_flag = 1;
        return false;
      }
      tc_fence_after();
      if (elect_one()) {
        issue_pv_wave(x, j, w);
        if (w + 1 == kWaves) {
          if (x == 1) umma_commit(v_free + (j & 1));
          if (j + 1 == n_x) umma_commit(o_full + x);
          if (j + 1 < n_x) {
            issue_qk(x, j + 1);
            if (x == 1) umma_commit(k_free + ((j + 1) & 1));
          }
        }
      }
      __syncwarp();
      return true;
    };
    auto waves_of = [&](auto item, int j) -> bool {
      bool good = step(item, std::integral_constant<int, 0>{}, j);
      if constexpr (kWaves >= 2) good = good && step(item, std::integral_constant<int, 1>{}, j);
      if constexpr (kWaves >= 4) {
        good = good && step(item, std::integral_constant<int, 2>{}, j);
        good = good && step(item, std::integral_constant<int, 3>{}, j);
      }
      return good;
    };
    // The fixed order  PV_0(j) QK_0(j+1) | PV_1(j) QK_1(j+1)  keeps the two items half a period
    // apart: the tensor pipe works on one while the other is in its softmax.  (Issuing whichever
    // item is ready first was measured: the items fall into step, both softmax groups run at
    // the same time and then both wait for the pipe, 285 against 249 us per layer.)
    for (int j = 0; j < nB && ok; ++j) {
      if (j < nA) ok = waves_of(std::integral_constant<int, 0>{}, j);
      if (ok) ok = waves_of(std::integral_constant<int, 1>{}, j);
    }
  } else {
    // ===== softmax: warps 0..7 own item 0, warps 8..15 item 1.  Within an item warp w and warp
    // w+4 share TMEM lanes (= query rows) 32*(w&3)..+31; the first owns columns 0..63 of S and
    // O, the second columns 64..127 =====
    const int x = warp >> 3;                      // item
    const int n_mine = x ? nB : nA;
    if (n_mine == 0 && pd.part >= 0 && pd.it[x].nrows > 0) {
      // this part holds none of the item's keys: a row sum of 0 tells the merge to skip it
      const int t = tid & 255;
      if (t < kTile) p.partials[pd.part * kPartSlotFloats + x * kPartItemFloats + int64_t(t) * kPartRow + kD + 1] = 0.f;
    }
    if (n_mine > 0) {
      const int t = tid & 255, row = t & 127, half = t >> 7;
      const uint32_t lane_addr = (uint32_t((warp & 3) * 32) << 16) + uint32_t(half * 64);
      const uint32_t tS = tmem + x * 128, tO = tmem + 256 + x * 128;
      const ItemDesc it = pd.it[x];
      float* my_half = s_half + x * 2 * kTile;
      const int bar_id = 1 + x;
      RowState st;
      bool failed = false;
      auto wait_all = [&](uint64_t* bar, int parity) {
        const bool bad = !wait_or_abort(bar, uint32_t(parity), abort_flag, p.wait_limit);
        if (softmax_sync_or(bar_id, bad)) failed = true;
        tc_fence_after();
        return !failed;
      };
      for (int j = 0; j < n_mine; ++j) {
        const bool bad = !wait_or_abort(s_full + x, uint32_t(j & 1), abort_flag, p.wait_limit);
        tc_fence_after();
        if (!softmax_tile<T>(tS, tO, lane_addr, row, half, p.qscale, j0 + j, j > 0, it.pos0, my_half, bar_id, st, bad,
                             flags + (warp & 15), uint32_t(j * kWaves), lane)) {
          failed = true;
          break;
        }
      }
      if (!failed && wait_all(o_full + x, 0)) {
        if (pd.part < 0)
          write_item<T>(tO, lane_addr, row, half, it, p.num_q_heads, p.out, my_half, bar_id, st, sQ + x * kOperandB);
        else
          write_partial(tO, lane_addr, row, half, p.partials + pd.part * kPartSlotFloats + x * kPartItemFloats,
                        my_half, bar_id, st);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicMax(p.status, KPX_ERR_DEVICE_TIMEOUT);
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

namespace {
// cuTensorMapEncodeTiled, looked up through the runtime so that the library carries no link
// dependency on the driver library.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}
// rank-n map of 16-bit elements, 128-byte swizzle; dims/box innermost first, strides in bytes
// for dimensions 1..n-1
bool make_map(CUtensorMap* map, int32_t dtype, const void* base, int rank, const cuuint64_t* dims,
              const cuuint64_t* strides_b, const cuuint32_t* box) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint32_t ones[4] = {1, 1, 1, 1};
  return fn(map, dtype == KPX_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
            cuuint32_t(rank), const_cast<void*>(base), dims, strides_b, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

// -1: cut underfilled calls (default); 0: never; 2..4: always, into that many parts (tests).
int g_prefill_split = -1;
// Test-only: polls before a bounded wait gives up, and the CTA whose first K tile never comes.
uint32_t g_prefill_wait_limit = kWaitLimit;
int g_prefill_withhold_cta = -1;

// Host side: pair list -> workspace, tensor maps, launch.  Returns KPX_ERR_UNIMPLEMENTED when
// the layout, dtype or scale is outside this path so that the caller can fall back to the
// streaming path.
int prefill_tc(void* out, const void* q, const void* k_pool, const void* v_pool, const kpx_kv_layout* layout,
               const int32_t* block_table, int32_t max_blocks_per_seq, const int32_t* cu_q_lens_host,
               const int32_t* start_pos_host, int32_t batch, int32_t num_q_heads, float scale, void* tile_area,
               int64_t tile_area_bytes, int32_t* status, cudaStream_t stream) {
  if (layout->dtype == KPX_F32 || layout->head_size != kD || layout->block_size != kBS || !block_table ||
      !(scale > 0.f))  // the row maximum is taken before scaling
    return KPX_ERR_UNIMPLEMENTED;
  // TMA: 16-byte aligned bases (strides are multiples of 16 bytes in every valid layout)
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 15)
    return KPX_ERR_UNIMPLEMENTED;
  const int kv_mul = num_q_heads / layout->num_kv_heads;
  const int32_t total_q = cu_q_lens_host[batch];
  // Items of one (sequence, KV head) in ascending position order, taken two at a time.
  std::vector<PairDesc> pairs;
  for (int32_t b = 0; b < batch; ++b) {
    const int32_t n = cu_q_lens_host[b + 1] - cu_q_lens_host[b];
    if (n <= 0) continue;
    for (int32_t kvh = 0; kvh < layout->num_kv_heads; ++kvh) {
      PairDesc pd{b, kvh, {{0, 0, 0, 0}, {0, 0, 0, 0}}, 0, 1 << 30, -1, 0};
      int held = 0;
      for (int32_t t0 = 0; t0 < n; t0 += kTile)
        for (int32_t h = kvh * kv_mul; h < (kvh + 1) * kv_mul; ++h) {
          const ItemDesc it{cu_q_lens_host[b] + t0, n - t0 < kTile ? n - t0 : kTile, start_pos_host[b] + t0, h};
          pd.it[held++] = it;
          if (held == 2) {
            pairs.push_back(pd);
            held = 0;
          }
        }
      if (held == 1) {  // a single item travels as it[1]
        pd.it[1] = pd.it[0];
        pd.it[0] = ItemDesc{0, 0, 0, 0};
        pairs.push_back(pd);
      }
    }
  }
  if (pairs.empty()) return KPX_OK;
  // longest first: the hardware hands CTAs out in order, so the short ones fill the tail
  auto cost = [](const PairDesc& d) {
    auto tiles = [](const ItemDesc& it) { return it.nrows > 0 ? (it.pos0 + it.nrows - 1) / kTile + 1 : 0; };
    return tiles(d.it[0]) + tiles(d.it[1]);
  };
  std::stable_sort(pairs.begin(), pairs.end(), [&](const PairDesc& a, const PairDesc& b) { return cost(a) > cost(b); });
  // One CTA per SM: a call with fewer pairs than a third of the SMs leaves most of them idle.
  // Its pairs are then cut along the keys into k = 3 or 4 parts that run side by side, each
  // leaving unnormalised rows in a slot, and a small kernel merges them (one 4096-token prompt
  // in chunks of 256: 927 -> 674 us per layer).  Measured and dropped: cutting in two when half
  // the SMs are idle (the slots, the merge launch and the fixed cost of a CTA, about 7 us, eat
  // the gain: 160 -> 205 us for one 2048-token prompt), and cutting the thin last wave of a
  // larger call (the parts queue behind the first wave anyway).
  std::vector<MergeDesc> merges;
  {
    const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
    const int n = int(pairs.size());
    const int tail = (n < sms || g_prefill_split >= 2) ? n : 0;
    int k = tail > 0 ? sms / tail : 1;
    if (k > 4) k = 4;
    if (k < 3) k = 1;
    if (g_prefill_split == 0) k = 1;            // test knob: never cut
    if (g_prefill_split >= 2) k = g_prefill_split > 4 ? 4 : g_prefill_split;  // test knob: always cut
    if (k >= 2) {
      std::vector<PairDesc> parts;
      int slot = 0;
      for (int i = n - tail; i < n; ++i) {
        const PairDesc& d = pairs[size_t(i)];
        auto tiles = [](const ItemDesc& it) { return it.nrows > 0 ? (it.pos0 + it.nrows - 1) / kTile + 1 : 0; };
        const int tb = tiles(d.it[1]), ta = tiles(d.it[0]);
        // every part gets at least one key tile of item 1; item 0 (never more tiles) may have none
        // in the last parts and then leaves a row sum of 0 there
        (void)ta;
        const int kk = tb < k ? tb : k;
        if (kk < 2 || slot + kk > kMaxPartSlots) {
          parts.push_back(d);
          continue;
        }
        MergeDesc m[2] = {};
        for (int j = 0; j < kk; ++j) {
          PairDesc c = d;
          c.tile0 = tb * j / kk;
          c.tile1 = tb * (j + 1) / kk;
          c.part = slot;
          for (int x = 0; x < 2; ++x) m[x].slot[j] = slot;
          ++slot;
          parts.push_back(c);
        }
        for (int x = 0; x < 2; ++x)
          if (d.it[x].nrows > 0) {
            m[x].it = d.it[x];
            m[x].parts = kk;
            m[x].x = x;
            merges.push_back(m[x]);
          }
      }
      pairs.resize(size_t(n - tail));
      std::stable_sort(parts.begin(), parts.end(), [&](const PairDesc& a, const PairDesc& b) {
        return (a.tile1 < (1 << 30) ? 2 * (a.tile1 - a.tile0) : cost(a)) > (b.tile1 < (1 << 30) ? 2 * (b.tile1 - b.tile0) : cost(b));
      });
      pairs.insert(pairs.end(), parts.begin(), parts.end());
    }
  }
  // layout of the area: [pair list][merge list][part slots]
  const int64_t pair_bytes = align256(int64_t(pairs.size()) * sizeof(PairDesc));
  const int64_t merge_bytes = align256(int64_t(merges.size()) * sizeof(MergeDesc));
  const int64_t slot_bytes = merges.empty() ? 0 : int64_t(kMaxPartSlots) * kPartSlotFloats * sizeof(float);
  if (pair_bytes + merge_bytes + slot_bytes > tile_area_bytes) return KPX_ERR_WORKSPACE_TOO_SMALL;

  CUtensorMap map_q, map_k, map_v;
  {
    // Q [total_q][heads][128]: box = 128 rows x one head x 64 elements
    const cuuint64_t dims[3] = {cuuint64_t(kD), cuuint64_t(num_q_heads), cuuint64_t(total_q)};
    const cuuint64_t strides[2] = {cuuint64_t(kD) * 2, cuuint64_t(num_q_heads) * kD * 2};
    const cuuint32_t box[3] = {64, 1, cuuint32_t(kTile)};
    if (!make_map(&map_q, layout->dtype, q, 3, dims, strides, box)) return KPX_ERR_UNIMPLEMENTED;
  }
  {
    // pool [blocks][kv heads][16 tokens][128] by its strides: box = one (block, head) tile x 64 elements
    const cuuint64_t nblocks = layout->num_blocks > 0 ? cuuint64_t(layout->num_blocks) : (cuuint64_t(1) << 24);
    const cuuint64_t dims[4] = {cuuint64_t(kD), cuuint64_t(kBS), cuuint64_t(layout->num_kv_heads), nblocks};
    const cuuint64_t strides[3] = {cuuint64_t(layout->token_stride) * 2, cuuint64_t(layout->head_stride) * 2,
                                   cuuint64_t(layout->block_stride) * 2};
    const cuuint32_t box[4] = {64, cuuint32_t(kBS), 1, 1};
    if (!make_map(&map_k, layout->dtype, k_pool, 4, dims, strides, box) ||
        !make_map(&map_v, layout->dtype, v_pool, 4, dims, strides, box))
      return KPX_ERR_UNIMPLEMENTED;
  }
  uint8_t* area = static_cast<uint8_t*>(tile_area);
  KPX_CUDA_TRY(cudaMemcpyAsync(area, pairs.data(), pairs.size() * sizeof(PairDesc), cudaMemcpyHostToDevice, stream));
  if (!merges.empty())
    KPX_CUDA_TRY(cudaMemcpyAsync(area + pair_bytes, merges.data(), merges.size() * sizeof(MergeDesc),
                                 cudaMemcpyHostToDevice, stream));
  PrefillParams p;
  p.partials = reinterpret_cast<float*>(area + pair_bytes + merge_bytes);
  p.out = out;
  p.block_table = block_table;
  p.pairs = static_cast<const PairDesc*>(tile_area);
  p.status = status;
  p.num_blocks = layout->num_blocks;
  p.max_blocks_per_seq = max_blocks_per_seq;
  p.num_q_heads = num_q_heads;
  p.kv_mul = kv_mul;
  p.qscale = scale * kLog2e;
  p.wait_limit = g_prefill_wait_limit;
  p.withhold_cta = g_prefill_withhold_cta;
  const unsigned grid = unsigned(pairs.size());
  auto launch = [&](auto kernel, std::atomic<uint64_t>* done_mask) -> int {
    // the shared-memory attribute is per device: set once per device (atomic bit mask of devices
    // 0..63, so that concurrent first calls and processes that alternate devices are safe)
    int dev = 0;
    KPX_CUDA_TRY(cudaGetDevice(&dev));
    const uint64_t bit = uint64_t(1) << (dev & 63);
    if (dev >= 64 || !(done_mask->load(std::memory_order_acquire) & bit)) {
      KPX_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      if (dev < 64) done_mask->fetch_or(bit, std::memory_order_release);
    }
    kernel<<<grid, kThreads, kSmemBytes, stream>>>(p, map_q, map_k, map_v);
    return cuda_status(cudaGetLastError());
  };
  static std::atomic<uint64_t> done_f16{0}, done_bf16{0};
  const int rc = layout->dtype == KPX_F16 ? launch(prefill_tc_kernel<__half>, &done_f16)
                                          : launch(prefill_tc_kernel<__nv_bfloat16>, &done_bf16);
  if (rc != KPX_OK || merges.empty()) return rc;
  const MergeDesc* md = reinterpret_cast<const MergeDesc*>(area + pair_bytes);
  if (layout->dtype == KPX_F16)
    prefill_merge_kernel<__half><<<dim3(unsigned(merges.size()), kTile / kMergeRowsPerCta), dim3(kD, kMergeRowLanes), 0, stream>>>(static_cast<__half*>(out), p.partials, md, num_q_heads);
  else
    prefill_merge_kernel<__nv_bfloat16><<<dim3(unsigned(merges.size()), kTile / kMergeRowsPerCta), dim3(kD, kMergeRowLanes), 0, stream>>>(static_cast<__nv_bfloat16*>(out), p.partials, md, num_q_heads);
  return cuda_status(cudaGetLastError());
}

// Bytes of the work area prefill_tc may need for a call with total_q query tokens.
int64_t prefill_tc_area_bytes(int32_t total_q, int32_t num_q_heads) {
  const int64_t h = num_q_heads > 0 ? num_q_heads : 1;
  // at most one pair entry per (128-row tile, head) and never more tiles than tokens, plus the
  // parts of a cut last wave; one merge entry per cut item; the part slots
  return align256((int64_t(total_q) + 1) * h * int64_t(sizeof(PairDesc)) + int64_t(kMaxPartSlots) * sizeof(PairDesc)) +
         align256(int64_t(2) * kMaxPartSlots * sizeof(MergeDesc)) +
         int64_t(kMaxPartSlots) * kPartSlotFloats * int64_t(sizeof(float));
}

}  // namespace kpx

// Test knob (not in the public header): makes a bounded wait of the tensor-core kernel run out
// without a faulting or endless kernel: CTA (`withhold_cta` & 0xffff) announces one tile to its
// barrier but never requests it (`withhold_cta` >> 16 = 0: K of its first key tile, 1: V of its
// first key tile, 2: K of its second key tile), and the waits give up after `wait_limit` polls
// (0: the default).
extern "C" __attribute__((visibility("default"))) void kpx_internal_set_prefill_fault(uint32_t wait_limit, int withhold_cta) {
  kpx::g_prefill_wait_limit = wait_limit ? wait_limit : kpx::kWaitLimit;
  kpx::g_prefill_withhold_cta = withhold_cta;
}
// Test knob (not in the public header): see g_prefill_split.
extern "C" __attribute__((visibility("default"))) void kpx_internal_set_prefill_split(int v) { kpx::g_prefill_split = v; }
