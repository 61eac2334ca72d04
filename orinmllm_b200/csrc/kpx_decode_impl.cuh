// Paged GQA decode attention for sm_100a: warp-granular split-KV streaming + merge.
//
// This header holds the kernel, its launch forms and the per-element-type dispatcher.  It is
// included by kpx_decode.cu (entry points) and by one translation unit per element type
// (kpx_decode_f16.cu, _bf16.cu, _f32.cu), each of which instantiates dispatch_decode<T> once, so
// that the three sets of kernels compile side by side.
//
// Work decomposition.  The cache of sequence b holds len_b tokens in blocks of 16.
// An "item" is one (sequence, kv head, query-head group) triple; its work is the
// sequence's blocks.  All blocks of all items are laid on one line (sequence-major)
// and cut into W equal contiguous ranges, one per *warp* of a persistent grid (one
// CTA per SM, 12 warps per CTA for 16-bit caches), so every warp streams the same
// number of bytes whatever the spread of sequence lengths.  A warp that covers an
// item completely writes its output directly; an item cut by a range boundary
// leaves one partial (running max, sum, un-normalised accumulator) per warp in the
// workspace, and the warp that delivers the item's last piece (an atomic counter per item,
// nobody waits) assembles the output; an item cut into more than 16 pieces is assembled in
// two levels, 16 warps' pieces at a time.  One launch.  A launch that the host can tell to
// be small (few blocks per warp) runs a second instantiation that cuts fewer, longer ranges.
//
// Each warp is its own producer and consumer: it owns two K and two V tile slots in
// shared memory, fetches the (block, kv head) tiles of its range through the block
// table with cp.async.bulk (the TMA engine, completion on per-slot mbarriers), and
// refills a slot the moment it has finished reading it -- the K slot right after
// the score pass, the V slot after the output pass.  There is no cross-warp
// synchronisation after the prologue.  A warp serves up to 4 query heads of the KV
// head from one tile read, so a K/V byte crosses HBM once per 4 query heads.  The
// math is fp32 on CUDA cores (packed fp32x2 FMAs); softmax is online with warp
// shuffles.  Every mbarrier wait is bounded; a wait that gives up raises the
// workspace status word and the warp retires.
#pragma once
#include <atomic>
#include <mutex>
#include <type_traits>

#include "kpx_common.cuh"

namespace kpx {
namespace decode {

constexpr int kD = 128;          // head size
constexpr int kBS = 16;          // tokens per block
constexpr int kMaxBatch = 512;   // sequences per launch (their block prefix lives in smem)
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeParams {
  void* out;
  const void* q;
  const uint8_t* k_pool;
  const uint8_t* v_pool;
  const int32_t* block_table;
  const int32_t* seq_lens;
  const int32_t* row_index;  // table row of each batch entry (nullptr: entry b uses row b)
  // Fused step (all nullptr otherwise): the new token of sequence b sits at position len_b (the
  // number of cached tokens); its q rows and k row are rotated here, its k / v rows are stored
  // into the pool and take part in the attention from registers.
  const void* k_new;   // [batch, kv_heads*128], not yet rotated
  const void* v_new;   // [batch, kv_heads*128]
  const float* sin_cache;
  const float* cos_cache;  // fp32 [max_pos, 128], read at pos*128 + 2j
  uint8_t* k_pool_w;
  uint8_t* v_pool_w;
  float* partials;
  int32_t* counters;  // one per item, zero between launches
  int32_t* status;
  int64_t block_stride_b, head_stride_b, token_stride_b;  // bytes
  int64_t num_blocks;
  int32_t max_blocks_per_seq, len_bias, batch;
  int32_t max_cached_tokens;  // most tokens a table row can address from the pool
  int32_t num_q_heads, num_kv_heads, kv_mul;
  int32_t head_groups;  // ceil(kv_mul / QH)
  int32_t partial_slots;  // slots of kPartialFloats floats in `partials`
  int32_t tile_contig;
  int32_t min_blocks_per_range, min_warps_per_sm;  // read by the small-launch form of the kernel only
  // Polls a bounded wait makes before it gives up (kWaitLimit), and, for the test of that path
  // only, the warp whose first tile request is announced to its barrier but never issued (-1: none).
  uint32_t wait_limit;
  int32_t withhold_worker;
  float qscale;  // softmax scale * log2(e)
  // A plan of this step (nullptr: none), see the layout below: what every launch of the step
  // would otherwise work out again in its prologue.
  const int32_t* plan;
};

// Plan of one decode step.  The launches of a step (one per layer) all see the same lengths and
// the same block table, so the block prefix over the sequences, every warp's starting point on
// the line of blocks and the id of its first block are the same for all of them; with a plan a
// CTA gets them with one load instead of three dependent ones (lengths, prefix and search, first
// block id).  int32 words: [0] mark, [1] batch, [2] warps the line is cut for, [3] items per
// sequence (kv heads x head groups), [4] an error to hand on (KPX_ERR_*), [8..8+kMaxBatch] the
// block prefix, then one entry of four words per warp: (sequence << 16 | item, block, tokens of
// the sequence, id of that block); sequence 0xffff = the warp has no blocks.
constexpr int32_t kPlanMark = 0x4b50504c;
constexpr int kPlanPrefixAt = 8, kPlanEntriesAt = kPlanPrefixAt + kMaxBatch + 8, kPlanEntryWords = 4;

template <typename T, int QH, int NW, int NS, int LPT>
struct Cfg {
  static constexpr int kEltB = sizeof(T);
  static constexpr int kTileB = kBS * kD * kEltB;  // one (block, head) tile of K or of V
  static constexpr int kWarps = NW;  // NS = K slots (and V slots) per warp
  static constexpr int kThreads = 32 * kWarps;
  static constexpr int kWarpRingB = 2 * NS * kTileB;  // K slots then V slots
  static constexpr int kOffBars = kWarps * kWarpRingB;
  static constexpr int kOffPrefix = kOffBars + kWarps * 2 * NS * 8;
  static constexpr int kOffP = kOffPrefix + (kMaxBatch + 1) * 4 + 12;
  static constexpr int kSmem = kOffP + kWarps * 2 * kBS * 4 * 4;  // two weight buffers per warp
  // Fused step only: per warp, the rotated query rows of the item's QH heads, the new token's
  // rotated K row and its V row (all of type T), and the id of the block the token goes to.
  static constexpr int kStageB = (QH + 2) * kD * kEltB + 16;
  static constexpr int kSmemFused = kSmem + kWarps * kStageB;
  // one workspace slot: QH accumulators of 128, then QH maxima, QH sums; padded so that
  // every slot starts on a 16-byte boundary (the assembling warp reads float4)
  static constexpr int kPartialFloats = QH * kD + 8;
};

// Tokens of sequence b that lie in the pool.  A length read from device memory that would reach
// past the sequence's table row is cut to the row (and reported by the prologue): the table is
// never read out of bounds.
__device__ __forceinline__ int seq_len_of(const DecodeParams& p, int b) {
  int len = (p.seq_lens ? p.seq_lens[b] : 0) + p.len_bias;
  if (p.block_table && len > p.max_cached_tokens) len = p.max_cached_tokens;
  return len < 0 ? 0 : len;
}
__device__ __forceinline__ int blocks_of(int len) { return (len + kBS - 1) / kBS; }

// prefix[b] = blocks of sequences 0..b-1 (prefix[0] = 0), worked out by the whole CTA; `report`:
// this CTA raises the status word for a length the table rows cannot hold.
__device__ __forceinline__ void block_prefix(const DecodeParams& p, int* prefix, int tid, int nthreads, int warp,
                                             int lane, bool report) {
  for (int b = tid; b < p.batch; b += nthreads) {
    prefix[b + 1] = blocks_of(seq_len_of(p, b));
    if (p.block_table && p.seq_lens && report && p.seq_lens[b] + p.len_bias > p.max_cached_tokens)
      atomicMax(p.status, KPX_ERR_INVALID_ARGUMENT);
  }
  if (tid == 0) prefix[0] = 0;
  __syncthreads();
  if (warp == 0) {  // inclusive scan in chunks of 32
    int carry = 0;
    for (int base = 0; base < p.batch; base += 32) {
      int i = base + lane;
      int v = i < p.batch ? prefix[i + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += n;
      }
      if (i < p.batch) prefix[i + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
}

// Position on the line of blocks: sequence b, sub-item (= kv_head*head_groups +
// head_group), block blk of the sequence.  kvh and the block-table row of b are
// kept alongside so the per-block path needs no division and no 64-bit multiply.
struct Cursor {
  int b, sub, blk, nblk, len, kvh;
  const int32_t* row;  // block-table row of sequence b (nullptr: identity table)
  __device__ __forceinline__ void refresh(const DecodeParams& p) {
    kvh = sub / p.head_groups;
    row = p.block_table
              ? p.block_table + int64_t(p.row_index ? p.row_index[b] : b) * p.max_blocks_per_seq
              : nullptr;
  }
  __device__ __forceinline__ void locate(const DecodeParams& p, const int* prefix, int64_t u) {
    const int per_seq = p.num_kv_heads * p.head_groups;
    int lo = 0, hi = p.batch;  // first b with prefix[b+1]*per_seq > u
    if (int64_t(prefix[p.batch]) * per_seq < (int64_t(1) << 31)) {
      // the whole line fits 31 bits (every launch but the very largest): 32-bit compares and one
      // 32-bit division instead of 64-bit ones; this runs before a warp's first tile request
      const uint32_t u32 = uint32_t(u), ps = uint32_t(per_seq);
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (uint32_t(prefix[mid + 1]) * ps > u32) hi = mid; else lo = mid + 1;
      }
      b = lo;
      nblk = prefix[b + 1] - prefix[b];
      const uint32_t r = u32 - uint32_t(prefix[b]) * ps;
      sub = int(r / uint32_t(nblk));
      blk = int(r - uint32_t(sub) * uint32_t(nblk));
    } else {
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (int64_t(prefix[mid + 1]) * per_seq > u) hi = mid; else lo = mid + 1;
      }
      b = lo;
      nblk = prefix[b + 1] - prefix[b];
      int64_t r = u - int64_t(prefix[b]) * per_seq;
      sub = int(r / nblk);
      blk = int(r - int64_t(sub) * nblk);
    }
    len = seq_len_of(p, b);
    refresh(p);
  }
  // one block forward; returns true when that left the current item
  __device__ __forceinline__ bool advance(const DecodeParams& p, const int* prefix) {
    if (++blk < nblk) return false;
    blk = 0;
    if (++sub == p.num_kv_heads * p.head_groups) {
      sub = 0;
      do { ++b; } while (b < p.batch && prefix[b + 1] == prefix[b]);
      if (b < p.batch) {
        nblk = prefix[b + 1] - prefix[b];
        len = seq_len_of(p, b);
      }
    }
    if (b < p.batch) refresh(p);
    return true;
  }
};

// The line of `total` blocks is cut into W contiguous ranges: the first `rem` ranges hold
// quot+1 blocks, the others quot (quot = total / W, rem = total % W).  Starts and owners need
// one multiply / one division by a small number instead of 64-bit divisions by W.
struct Split {
  int64_t quot, rem;
  __device__ __forceinline__ int64_t start(int64_t c) const { return c * quot + (c < rem ? c : rem); }
  __device__ __forceinline__ int64_t owner(int64_t u) const {
    const int64_t big = rem * (quot + 1);  // blocks held by the ranges of quot+1
    if (u < big) return (big >> 31) ? u / (quot + 1) : int64_t(uint32_t(u) / uint32_t(quot + 1));
    const int64_t v = u - big;
    return rem + ((v >> 31) || (quot >> 31) ? v / quot : int64_t(uint32_t(v) / uint32_t(quot)));
  }
};

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Fused step, start of an item: rotates the new token's query rows of the item's QH heads at
// position `pos` and leaves them, rounded to T, in the warp's staging area; with `with_kv` (the
// warp's segment reaches the end of the item, so it will also account for the new token) the
// rotated K row, the V row and the id of the block that takes the token follow.  Half-split
// pairs (j, j + 64), sin/cos read at pos*128 + 2j, products rounded separately and one rounding
// to T: the bits rope_append_kernel stores.  Kept out of line so that the streaming loop's
// register allocation is that of the plain kernel; the caller brackets it with __syncwarp().
template <typename T, int QH>
__device__ __noinline__ void stage_new_token(const T* q_kv_group, int hg, int kv_mul, const T* k_row,
                                             const uint8_t* v_row, bool with_kv, const float* sin_row,
                                             const float* cos_row, const int32_t* table_entry,
                                             int identity_id, uint8_t* stage, int lane) {
  constexpr int E = Elt<T>::kPer16B;
  constexpr int G = kD / 2 / E;  // 16-byte pair groups per row
  constexpr int kRowB = kD * int(sizeof(T));
  const int rows = QH + (with_kv ? 1 : 0);
  for (int task = lane; task < rows * G; task += 32) {
    const int r = task / G, g = task - r * G;
    const int hq = hg * QH + r;
    const T* src = r < QH ? q_kv_group + (hq < kv_mul ? hq : 0) * kD : k_row;
    float lo[E], hi[E];
    Elt<T>::unpack(__ldg(reinterpret_cast<const uint4*>(src + g * E)), lo);
    Elt<T>::unpack(__ldg(reinterpret_cast<const uint4*>(src + kD / 2 + g * E)), hi);
    __align__(16) T lo_out[E];
    __align__(16) T hi_out[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float sn = __ldg(sin_row + 2 * (g * E + e)), cs = __ldg(cos_row + 2 * (g * E + e));
      lo_out[e] = Elt<T>::from_float(__fsub_rn(__fmul_rn(lo[e], cs), __fmul_rn(hi[e], sn)));
      hi_out[e] = Elt<T>::from_float(__fadd_rn(__fmul_rn(lo[e], sn), __fmul_rn(hi[e], cs)));
    }
    uint8_t* dst = stage + r * kRowB;
    *reinterpret_cast<uint4*>(dst + g * 16) = *reinterpret_cast<const uint4*>(lo_out);
    *reinterpret_cast<uint4*>(dst + kRowB / 2 + g * 16) = *reinterpret_cast<const uint4*>(hi_out);
  }
  if (with_kv) {
    for (int task = lane; task < kRowB / 16; task += 32)
      *reinterpret_cast<uint4*>(stage + (QH + 1) * kRowB + task * 16) =
          __ldg(reinterpret_cast<const uint4*>(v_row) + task);
    if (lane == 0)
      *reinterpret_cast<int32_t*>(stage + (QH + 2) * kRowB) = table_entry ? __ldg(table_entry) : identity_id;
  }
}

// kSmall: the form launched when the host can tell from the batch size and the table width that
// the launch has only a few blocks per warp (a short batch, or one KV head of one long
// sequence).  It cuts the line into fewer, longer ranges: every piece of a cut item costs a
// partial and a share of the assembly, and a range of a block or two is all prologue.  Warps
// are then numbered CTA-minor so that the active ones stay spread over all SMs.  The policy
// is compiled out of the other form, whose code is the same as without it.
template <typename T, int QH, int NW, int NS, int LPT, bool kSmall = false, int CPS = 1, bool kFused = false>
__global__ void __launch_bounds__(Cfg<T, QH, NW, NS, LPT>::kThreads, CPS)
paged_decode_kernel(const DecodeParams p) {
  using C = Cfg<T, QH, NW, NS, LPT>;
  constexpr int E = Elt<T>::kPer16B;  // elements per 16-byte vector
  // LPT lanes share one token row: each owns DPT = 128/LPT dims; a warp covers TG = 32/LPT
  // token rows per pass and R = 16/TG passes per block.
  constexpr int TG = 32 / LPT, R = kBS / TG, DPT = kD / LPT, HP = DPT / 2;
  constexpr int NCH = DPT / E;        // 16-byte chunks per thread per row
  constexpr int NV = (QH == 4) ? 2 : 1;  // finished scores per thread per block
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBars) + warp * 2 * NS;  // K slots, V slots
  int* prefix = reinterpret_cast<int*>(smem + C::kOffPrefix);
  uint8_t* ring = smem + warp * C::kWarpRingB;
  float* p_s = reinterpret_cast<float*>(smem + C::kOffP) + warp * (2 * kBS * 4);  // two buffers
  uint8_t* stage = smem + C::kSmem + warp * C::kStageB;  // fused step only

  // ---- prologue: block prefix over sequences (whole CTA), this warp's barriers ----
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < 2 * NS; ++s) mbar_init(bars + s, 1);
    mbar_fence_init();
  }
  // With a plan of the step the prefix and this warp's starting point come from it: one round
  // trip to global memory instead of lengths -> prefix -> search -> first block id.
  bool planned = false;
  int4 plan_entry = make_int4(0, 0, 0, 0);
  if constexpr (!kSmall && !kFused) {
    if (p.plan) {
      // header, this warp's entry and the prefix are requested together (a plan buffer always
      // holds kMaxSms x 16 entries and kMaxBatch + 1 prefix words, whatever was planned); what
      // the header says decides afterwards whether they are used
      const int4 h = __ldg(reinterpret_cast<const int4*>(p.plan));
      const int32_t plan_error = __ldg(p.plan + 4);
      plan_entry = __ldg(reinterpret_cast<const int4*>(p.plan + kPlanEntriesAt) + (blockIdx.x * C::kWarps + warp));
      for (int b = tid; b <= p.batch; b += C::kThreads) prefix[b] = __ldg(p.plan + kPlanPrefixAt + b);
      planned = h.x == kPlanMark && h.y == p.batch && h.z == int(gridDim.x) * C::kWarps &&
                h.w == p.num_kv_heads * p.head_groups;
      if (planned && blockIdx.x == 0 && tid == 0 && plan_error != 0) atomicMax(p.status, plan_error);
      __syncthreads();
    }
  }
  if (!planned) block_prefix(p, prefix, tid, C::kThreads, warp, lane, blockIdx.x == 0);
  // a sequence without tokens gets zeros (no warp ever visits it); CTAs share the rows.
  // In the fused step its only token is the new one: every head's output is that token's V
  // row, and its rotated K (position 0: unchanged) and V rows go to slot 0 of its first block.
  for (int b = blockIdx.x; b < p.batch; b += gridDim.x) {
    if (prefix[b + 1] != prefix[b]) continue;
    T* o = static_cast<T*>(p.out) + int64_t(b) * p.num_q_heads * kD;
    if (!kFused) {
      for (int e = tid; e < p.num_q_heads * kD; e += C::kThreads) o[e] = Elt<T>::from_float(0.f);
      continue;
    }
    const T* vn = static_cast<const T*>(p.v_new) + int64_t(b) * p.num_kv_heads * kD;
    for (int e = tid; e < p.num_q_heads * kD; e += C::kThreads) o[e] = vn[(e / kD / p.kv_mul) * kD + e % kD];
    const int32_t* row = p.block_table ? p.block_table + int64_t(p.row_index ? p.row_index[b] : b) * p.max_blocks_per_seq : nullptr;
    int id = row ? row[0] : 0;
    if (id < 0 || (p.num_blocks > 0 && id >= p.num_blocks)) {
      if (tid == 0) atomicMax(p.status, KPX_ERR_INVALID_ARGUMENT);
      continue;
    }
    const T* kn = static_cast<const T*>(p.k_new) + int64_t(b) * p.num_kv_heads * kD;
    for (int e = tid; e < p.num_kv_heads * kD; e += C::kThreads) {
      const int h = e / kD, d = e % kD, j = d & (kD / 2 - 1);
      const float lo = Elt<T>::to_float(kn[h * kD + j]), hi = Elt<T>::to_float(kn[h * kD + kD / 2 + j]);
      const float sn = __ldg(p.sin_cache + 2 * j), cs = __ldg(p.cos_cache + 2 * j);
      const float r = d >= kD / 2 ? __fadd_rn(__fmul_rn(lo, sn), __fmul_rn(hi, cs))
                                  : __fsub_rn(__fmul_rn(lo, cs), __fmul_rn(hi, sn));
      const int64_t off = int64_t(id) * p.block_stride_b + int64_t(h) * p.head_stride_b + int64_t(d) * C::kEltB;
      *reinterpret_cast<T*>(p.k_pool_w + off) = Elt<T>::from_float(r);
      *reinterpret_cast<T*>(p.v_pool_w + off) = vn[e];
    }
  }
  const int64_t total = int64_t(prefix[p.batch]) * p.num_kv_heads * p.head_groups;
  int64_t W_ = int64_t(gridDim.x) * C::kWarps;
  int64_t worker_ = int64_t(blockIdx.x) * C::kWarps + warp;
  if constexpr (kSmall) {
    if (total < W_ * p.min_blocks_per_range) {
      int64_t w = total / p.min_blocks_per_range;
      const int64_t floor_w = int64_t(gridDim.x) * (C::kWarps < p.min_warps_per_sm ? C::kWarps : p.min_warps_per_sm);
      if (w < floor_w) w = floor_w;
      if (w < 1) w = 1;
      if (w < W_) W_ = w;
      worker_ = int64_t(warp) * gridDim.x + blockIdx.x;
      if (worker_ >= W_) return;  // nothing below synchronises across warps
    }
  }
  const int64_t W = W_;
  const int64_t worker = worker_;
  Split split;
  if (total < (int64_t(1) << 31)) {  // (W is at most a few thousand)
    split.quot = int64_t(uint32_t(total) / uint32_t(W));
  } else {
    split.quot = total / W;
  }
  split.rem = total - split.quot * W;
  const int64_t u0 = split.start(worker), u1 = split.start(worker + 1);
  if (u0 >= u1) return;  // nothing below synchronises across warps
  const int n = int(u1 - u0);

  const int tg = lane / LPT;  // token group: rows r*TG + tg
  const int sub = lane % LPT;  // owns DPT of the 128 dims
  // Register r of the score pass holds token (r ^ perm)*4 + tg: the lane-dependent
  // order lets the cross-lane halving below keep/send fixed registers.
  const int perm = sub >> 1;
  const int my_j0 = (QH == 4) ? (sub & 1) * 2 : (QH == 2 ? (sub & 1) : 0);
  const bool hi_lane = (sub & 1) != 0;
  // byte offset of this thread's chunk c inside a row of a tile
  int coff[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) coff[c] = (c * (kD / NCH) + sub * E) * C::kEltB;

  // ---- producer side: block ids and bulk copies of this warp's own range ----
  // One cursor walks the range NS blocks ahead of the consumer.  The K tile of a block
  // is requested when a K slot frees up; its V tile is requested one step later (the
  // output pass trails the score pass by one block), reusing the source offset and
  // row count remembered from the K request.
  Cursor cur;  // consumer side: first block of the current segment
  if (planned) {
    cur.b = plan_entry.x >> 16;
    cur.sub = plan_entry.x & 0xffff;
    cur.blk = plan_entry.y;
    cur.len = plan_entry.z;
    cur.nblk = prefix[cur.b + 1] - prefix[cur.b];
    cur.refresh(p);
  } else {
    cur.locate(p, prefix, u0);
  }
  // The first item's query rows are requested here, before the first block id and the first
  // tiles, so that their latency (DRAM if nothing brought them to L2) runs under those.
  uint4 q_first[kFused ? 1 : QH][kFused ? 1 : NCH];
  if constexpr (!kFused) {
    const int hg0 = cur.sub - cur.kvh * p.head_groups;
    const T* qrow0 = static_cast<const T*>(p.q) + int64_t(cur.b) * p.num_q_heads * kD;
#pragma unroll
    for (int j = 0; j < QH; ++j) {
      const int hq = hg0 * QH + j;
      const T* qh = qrow0 + int64_t(cur.kvh * p.kv_mul + (hq < p.kv_mul ? hq : 0)) * kD;
#pragma unroll
      for (int c = 0; c < NCH; ++c)
        q_first[j][c] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(qh) + coff[c]));
    }
  }
  Cursor pc = cur;      // producer side: walks the range NS blocks ahead
  int pc_id;            // block id at pc (loaded one step before it is needed)
  int64_t last_off = 0; // byte offset of the last requested block's (block, kv head) tile
  int last_rows = kBS;  // its number of existing rows (strided layout only)
  int k_issued = 0, v_issued = 0;
  auto load_id = [&]() -> int {
    int id = pc.row ? __ldg(pc.row + pc.blk) : pc.blk;
    if (id < 0 || (p.num_blocks > 0 && id >= p.num_blocks)) {
      if (lane == 0) atomicMax(p.status, KPX_ERR_INVALID_ARGUMENT);
      id = 0;
    }
    return id;
  };
  // request one tile (callers have __syncwarp'ed after the last read of the slot)
  auto copy_tile = [&](const uint8_t* pool, int64_t off, int rows, int slot_index, bool withhold = false) {
    uint64_t* bar = bars + slot_index;
    uint8_t* dst = ring + slot_index * C::kTileB;
    if (p.tile_contig) {
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, C::kTileB);
        if (!withhold) bulk_g2s(dst, pool + off, C::kTileB, bar);
      }
    } else {
      // strided rows (the reference's token-major cache): one bulk copy per existing row
      constexpr int kRowB = kD * C::kEltB;
      if (lane == 0) mbar_arrive_expect_tx(bar, uint32_t(rows) * kRowB);
      __syncwarp();
      if (lane < rows) bulk_g2s(dst + lane * kRowB, pool + off + int64_t(lane) * p.token_stride_b, kRowB, bar);
    }
  };
  auto issue_k = [&](int slot) {  // K tile of the block at pc; then step pc
    last_off = int64_t(pc_id) * p.block_stride_b + int64_t(pc.kvh) * p.head_stride_b;
    last_rows = min(kBS, pc.len - pc.blk * kBS);
    copy_tile(p.k_pool, last_off, last_rows, slot, k_issued == 0 && worker == p.withhold_worker);
    ++k_issued;
    pc.advance(p, prefix);
    if (k_issued < n) pc_id = load_id();
  };
  auto issue_v = [&](int slot) {  // V tile of the block whose K tile was requested last
    copy_tile(p.v_pool, last_off, last_rows, NS + slot);
    ++v_issued;
  };
  if (planned) {
    pc_id = plan_entry.w;
    if (pc_id < 0 || (p.num_blocks > 0 && pc_id >= p.num_blocks)) {
      if (lane == 0) atomicMax(p.status, KPX_ERR_INVALID_ARGUMENT);
      pc_id = 0;
    }
  } else {
    pc_id = load_id();
  }
#pragma unroll
  for (int k = 0; k < NS; ++k) {
    if (k < n) {
      issue_k(k);
      issue_v(k);
    }
  }

  // ---- consumer state ----
  float2 q2[QH][HP];
  float2 acc[QH][HP];
  float m_run[NV], l_run[NV];

  // blocks_left: blocks of the warp's range from the item's first block in it onwards;
  // first_tag: the warp's first item, whose query rows were requested in the prologue
  auto begin_item = [&](int blocks_left, auto first_tag) {
    constexpr bool kFirst = decltype(first_tag)::value;
    const int hg = cur.sub - cur.kvh * p.head_groups;
    const T* qrow = static_cast<const T*>(p.q) + int64_t(cur.b) * p.num_q_heads * kD;
    if constexpr (kFused) {
      const int seg = min(blocks_left, cur.nblk - cur.blk);
      const bool ends_item = cur.blk + seg == cur.nblk;
      __syncwarp();  // the previous item's readers of the staging area are done
      stage_new_token<T, QH>(
          qrow + int64_t(cur.kvh) * p.kv_mul * kD, hg, p.kv_mul,
          static_cast<const T*>(p.k_new) + (int64_t(cur.b) * p.num_kv_heads + cur.kvh) * kD,
          static_cast<const uint8_t*>(p.v_new) + (int64_t(cur.b) * p.num_kv_heads + cur.kvh) * (kD * C::kEltB),
          ends_item, p.sin_cache + int64_t(cur.len) * kD, p.cos_cache + int64_t(cur.len) * kD,
          cur.row ? cur.row + cur.len / kBS : nullptr, cur.len / kBS, stage, lane);
      __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < QH; ++j) {
      const int hq = hg * QH + j;
      const bool valid = hq < p.kv_mul;
      const T* qh = qrow + int64_t(cur.kvh * p.kv_mul + (valid ? hq : 0)) * kD;
      const float sc = valid ? p.qscale : 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        float f[E];
        uint4 raw;
        if constexpr (kFused)  // rotated at the new token's position, rounded to T
          raw = *reinterpret_cast<const uint4*>(stage + j * (kD * C::kEltB) + coff[c]);
        else if constexpr (kFirst)
          raw = q_first[j][c];
        else
          raw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(qh) + coff[c]));
        Elt<T>::unpack(raw, f);
#pragma unroll
        for (int e = 0; e < E; e += 2)
          q2[j][(c * E + e) / 2] = make_float2(f[e] * sc, f[e + 1] * sc);
      }
#pragma unroll
      for (int i = 0; i < HP; ++i) acc[j][i] = make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) { m_run[k] = -INFINITY; l_run[k] = 0.f; }
  };

  // out += p * V for the block whose V tile is at vt and whose weights are in pb.
  // kFull: all 16 tokens exist (no predicates).
  auto pv_pass = [&](const uint8_t* vt, const float* pb, int nvalid, auto full_tag) {
    constexpr bool kFull = decltype(full_tag)::value;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int tok = r * TG + tg;
      if (kFull || tok < nvalid) {
        float vf[DPT];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint4 raw = *reinterpret_cast<const uint4*>(vt + tok * (kD * C::kEltB) + coff[c]);
          Elt<T>::unpack(raw, vf + c * E);
        }
        float pj[4];
        if (QH == 4) {
          float4 t4 = *reinterpret_cast<const float4*>(pb + tok * 4);
          pj[0] = t4.x; pj[1] = t4.y; pj[2] = t4.z; pj[3] = t4.w;
        } else if (QH == 2) {
          float2 t2 = *reinterpret_cast<const float2*>(pb + tok * 4);
          pj[0] = t2.x; pj[1] = t2.y;
        } else {
          pj[0] = pb[tok * 4];
        }
#pragma unroll
        for (int j = 0; j < QH; ++j) {
          const float2 pp = make_float2(pj[j], pj[j]);
#pragma unroll
          for (int d = 0; d < HP; ++d)
            acc[j][d] = __ffma2_rn(pp, make_float2(vf[2 * d], vf[2 * d + 1]), acc[j][d]);
        }
      }
    }
  };

  auto end_item = [&](const Cursor& item, bool whole_item, int64_t partial_slot, int64_t item_start,
                      bool has_item_end) {
    const int hg = item.sub - item.kvh * p.head_groups;
    // totals over the 4 token groups (every lane ends with the sums of its 16 dims)
#pragma unroll
    for (int j = 0; j < QH; ++j)
#pragma unroll
      for (int i = 0; i < HP; ++i) {
        float2 a = acc[j][i];
#pragma unroll
        for (int m = LPT; m < 32; m <<= 1) {
          a.x += __shfl_xor_sync(0xffffffffu, a.x, m);
          a.y += __shfl_xor_sync(0xffffffffu, a.y, m);
        }
        acc[j][i] = a;
      }
    float mh[QH], lh[QH];  // running max and sum of every head, in every lane
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float l = l_run[k];
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      l_run[k] = l;
    }
    if (QH == 4) {
      float om0 = __shfl_xor_sync(0xffffffffu, m_run[0], 1), om1 = __shfl_xor_sync(0xffffffffu, m_run[NV - 1], 1);
      float ol0 = __shfl_xor_sync(0xffffffffu, l_run[0], 1), ol1 = __shfl_xor_sync(0xffffffffu, l_run[NV - 1], 1);
      mh[0] = hi_lane ? om0 : m_run[0];           lh[0] = hi_lane ? ol0 : l_run[0];
      mh[1 % QH] = hi_lane ? om1 : m_run[NV - 1]; lh[1 % QH] = hi_lane ? ol1 : l_run[NV - 1];
      mh[2 % QH] = hi_lane ? m_run[0] : om0;      lh[2 % QH] = hi_lane ? l_run[0] : ol0;
      mh[3 % QH] = hi_lane ? m_run[NV - 1] : om1; lh[3 % QH] = hi_lane ? l_run[NV - 1] : ol1;
    } else if (QH == 2) {
      float om = __shfl_xor_sync(0xffffffffu, m_run[0], 1), ol = __shfl_xor_sync(0xffffffffu, l_run[0], 1);
      mh[0] = hi_lane ? om : m_run[0];      lh[0] = hi_lane ? ol : l_run[0];
      mh[1 % QH] = hi_lane ? m_run[0] : om; lh[1 % QH] = hi_lane ? l_run[0] : ol;
    } else {
      mh[0] = m_run[0];
      lh[0] = l_run[0];
    }
    if (kFused && has_item_end) {
      // Fused step: this piece ends the item, so it also carries the new token (position
      // item.len, not in the pool yet).  Its rotated K row and its V row were staged when the
      // item began; every token group computes the same update for its dims.
      constexpr int kRowB = kD * C::kEltB;
      float kr[DPT], vf[DPT];
      uint4 kraw[NCH], vraw[NCH];
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        kraw[c] = *reinterpret_cast<const uint4*>(stage + QH * kRowB + coff[c]);
        vraw[c] = *reinterpret_cast<const uint4*>(stage + (QH + 1) * kRowB + coff[c]);
        Elt<T>::unpack(kraw[c], kr + c * E);
        Elt<T>::unpack(vraw[c], vf + c * E);
      }
#pragma unroll
      for (int j = 0; j < QH; ++j) {
        float sj = 0.f;
#pragma unroll
        for (int d = 0; d < HP; ++d) sj = fmaf(q2[j][d].x, kr[2 * d], fmaf(q2[j][d].y, kr[2 * d + 1], sj));
#pragma unroll
        for (int m = 1; m < LPT; m <<= 1) sj += __shfl_xor_sync(0xffffffffu, sj, m);
        const float m_new = fmaxf(mh[j], sj);
        const float a = fast_exp2(mh[j] - m_new), pw = fast_exp2(sj - m_new);
        mh[j] = m_new;
        lh[j] = lh[j] * a + pw;
#pragma unroll
        for (int d = 0; d < HP; ++d) {
          acc[j][d].x = fmaf(pw, vf[2 * d], acc[j][d].x * a);
          acc[j][d].y = fmaf(pw, vf[2 * d + 1], acc[j][d].y * a);
        }
      }
      // append: the first head group's warp stores the rows (token group 0 the K row, the last
      // token group the V row) into the block that holds position item.len
      if (hg == 0 && (tg == 0 || tg == TG - 1)) {
        const int id = *reinterpret_cast<const int32_t*>(stage + (QH + 2) * kRowB);
        if (id < 0 || (p.num_blocks > 0 && id >= p.num_blocks)) {
          if (sub == 0) atomicMax(p.status, KPX_ERR_INVALID_ARGUMENT);
        } else {
          const int64_t off = int64_t(id) * p.block_stride_b + int64_t(item.kvh) * p.head_stride_b +
                              int64_t(item.len % kBS) * p.token_stride_b;
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            if (tg == 0) *reinterpret_cast<uint4*>(p.k_pool_w + off + coff[c]) = kraw[c];
            if (tg == TG - 1) *reinterpret_cast<uint4*>(p.v_pool_w + off + coff[c]) = vraw[c];
          }
        }
      }
    }
    // token group tg writes the heads j with j % TG == tg (all groups hold the same sums)
#pragma unroll
    for (int j = 0; j < QH; ++j) {
      const int hq = hg * QH + j;
      if (tg == (j % TG) && hq < p.kv_mul) {
        if (whole_item) {
          uint8_t* o = reinterpret_cast<uint8_t*>(static_cast<T*>(p.out) + int64_t(item.b) * p.num_q_heads * kD +
                                                  int64_t(item.kvh * p.kv_mul + hq) * kD);
          const float inv = 1.f / lh[j];
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            __align__(16) T tmp[E];
#pragma unroll
            for (int e = 0; e < E; e += 2) {
              float2 a = acc[j][(c * E + e) / 2];
              tmp[e] = Elt<T>::from_float(a.x * inv);
              tmp[e + 1] = Elt<T>::from_float(a.y * inv);
            }
            *reinterpret_cast<uint4*>(o + coff[c]) = *reinterpret_cast<const uint4*>(tmp);
          }
        } else {
          float* ps = p.partials + partial_slot * C::kPartialFloats;
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int e = 0; e < E; e += 2)
              *reinterpret_cast<float2*>(ps + j * kD + coff[c] / C::kEltB + e) = acc[j][(c * E + e) / 2];
          if (sub == 0) {
            ps[QH * kD + j] = mh[j];
            ps[QH * kD + QH + j] = lh[j];
          }
        }
      }
    }
    if (whole_item) return;
    // The item is cut by a range boundary.  Publish this piece, then count it; the warp
    // that brings the count up to the number of pieces assembles the item from all of
    // them (nobody waits: whoever arrives last does the work) and resets the counter.
    __syncwarp();  // every lane's piece is ordered before lane 0's release below
    // every warp between the owners of the item's first and last block holds a piece of it
    const int64_t c_first = split.owner(item_start), c_last = split.owner(item_start + item.nblk - 1);
    const int pieces = int(c_last - c_first) + 1;
    // release our writes, acquire the other arrivals' (device scope, cumulative over the warp);
    // true in the warp that arrives last, which also resets the counter
    auto arrive_last = [&](int* cnt, int expected) -> bool {
      int prev = 0;
      if (lane == 0)
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(prev) : "l"(cnt) : "memory");
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev != expected - 1) return false;
      if (lane == 0) *cnt = 0;
      __syncwarp();
      return true;
    };
    auto slot_of = [&](int64_t c) {  // only the first piece can be a "tail" slot
      return p.partials + ((c == c_first) ? 2 * c + 1 : 2 * c) * C::kPartialFloats;
    };
    // Merges n slots into the item's output rows (dst == nullptr) or into one unnormalised slot.
    // Token group tg handles the heads j with j % TG == tg, lane `sub` its DPT dims.  The
    // weights 2^(m_c - M) need the overall maximum first; with M known every slot's term is
    // independent, so the loads of the accumulation loop can be in flight together.
    // The LPT lanes of a token group walk the head loop together (same j, same trip count);
    // other groups may be elsewhere, so the shuffles name only the group's own lanes.
    const uint32_t group_mask = (LPT == 32 ? 0xffffffffu : ((1u << LPT) - 1u)) << (tg * LPT);
    auto merge = [&](int64_t n, auto slot_fn, float* dst) {
      for (int j = tg; j < QH; j += TG) {
        const int hq = hg * QH + j;
        if (hq >= p.kv_mul) continue;
        float M = -INFINITY;
        for (int64_t i = sub; i < n; i += LPT) M = fmaxf(M, __ldcg(slot_fn(i) + QH * kD + j));
#pragma unroll
        for (int m = 1; m < LPT; m <<= 1) M = fmaxf(M, __shfl_xor_sync(group_mask, M, m));
        float L = 0.f;
        for (int64_t i = sub; i < n; i += LPT) {
          const float* ps = slot_fn(i);
          L += __ldcg(ps + QH * kD + QH + j) * fast_exp2(__ldcg(ps + QH * kD + j) - M);
        }
#pragma unroll
        for (int m = 1; m < LPT; m <<= 1) L += __shfl_xor_sync(group_mask, L, m);
        float O[DPT];
#pragma unroll
        for (int e = 0; e < DPT; ++e) O[e] = 0.f;
#pragma unroll 4
        for (int64_t i = 0; i < n; ++i) {
          const float* ps = slot_fn(i);
          const float w = fast_exp2(__ldcg(ps + QH * kD + j) - M);
#pragma unroll
          for (int k = 0; k < DPT / 4; ++k) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(ps + j * kD + coff[(k * 4) / E] / C::kEltB + (k * 4) % E));
            O[4 * k + 0] = fmaf(v.x, w, O[4 * k + 0]);
            O[4 * k + 1] = fmaf(v.y, w, O[4 * k + 1]);
            O[4 * k + 2] = fmaf(v.z, w, O[4 * k + 2]);
            O[4 * k + 3] = fmaf(v.w, w, O[4 * k + 3]);
          }
        }
        if (dst) {
#pragma unroll
          for (int k = 0; k < DPT / 4; ++k)
            *reinterpret_cast<float4*>(dst + j * kD + coff[(k * 4) / E] / C::kEltB + (k * 4) % E) =
                make_float4(O[4 * k + 0], O[4 * k + 1], O[4 * k + 2], O[4 * k + 3]);
          if (sub == 0) {
            dst[QH * kD + j] = M;
            dst[QH * kD + QH + j] = L;
          }
        } else {
          uint8_t* o = reinterpret_cast<uint8_t*>(static_cast<T*>(p.out) + int64_t(item.b) * p.num_q_heads * kD +
                                                  int64_t(item.kvh * p.kv_mul + hq) * kD);
          const float inv = 1.f / L;
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            __align__(16) T tmp[E];
#pragma unroll
            for (int e = 0; e < E; ++e) tmp[e] = Elt<T>::from_float(O[c * E + e] * inv);
            *reinterpret_cast<uint4*>(o + coff[c]) = *reinterpret_cast<const uint4*>(tmp);
          }
        }
      }
    };
    int* item_cnt = p.counters + (item.b * (p.num_kv_heads * p.head_groups) + item.sub);
    // An item cut into many pieces (one very long sequence) is assembled in two levels so that
    // no single warp reads them all: the pieces of kGroup consecutive warps are merged by the
    // last of them to arrive into one slot of a second area, and the last group to finish
    // merges those.  The second area sits at the end of the slot array: [group slots][one
    // slot of group counters]; it is used only if the array has room for it.
    constexpr int kGroup = 16, kFlatMax = 16;  // kFlatMax >= kGroup: a group then never holds more than two grouped items
    const int64_t W_all = int64_t(gridDim.x) * C::kWarps;
    const int64_t n_groups = (W_all + kGroup - 1) / kGroup;
    const int64_t group_base = int64_t(p.partial_slots) - 1 - 2 * n_groups;  // first group slot
    if (pieces <= kFlatMax || group_base < 2 * W_all || 2 * n_groups * 4 > int64_t(C::kPartialFloats) * 4) {
      if (!arrive_last(item_cnt, pieces)) return;
      // a handful of pieces: one pass with a running maximum
      for (int j = tg; j < QH; j += TG) {
        const int hq = hg * QH + j;
        if (hq >= p.kv_mul) continue;
        float M = -INFINITY, L = 0.f;
        float O[DPT];
#pragma unroll
        for (int e = 0; e < DPT; ++e) O[e] = 0.f;
#pragma unroll 2
        for (int64_t c = c_first; c <= c_last; ++c) {
          const float* ps = slot_of(c);
          const float mw = __ldcg(ps + QH * kD + j), lw = __ldcg(ps + QH * kD + QH + j);
          float4 v[DPT / 4];
#pragma unroll
          for (int k = 0; k < DPT / 4; ++k)
            v[k] = __ldcg(reinterpret_cast<const float4*>(ps + j * kD + coff[(k * 4) / E] / C::kEltB + (k * 4) % E));
          const float Mn = fmaxf(M, mw);
          const float a = fast_exp2(M - Mn), bsc = fast_exp2(mw - Mn);
          L = L * a + lw * bsc;
#pragma unroll
          for (int k = 0; k < DPT / 4; ++k) {
            O[4 * k + 0] = O[4 * k + 0] * a + v[k].x * bsc;
            O[4 * k + 1] = O[4 * k + 1] * a + v[k].y * bsc;
            O[4 * k + 2] = O[4 * k + 2] * a + v[k].z * bsc;
            O[4 * k + 3] = O[4 * k + 3] * a + v[k].w * bsc;
          }
          M = Mn;
        }
        uint8_t* o = reinterpret_cast<uint8_t*>(static_cast<T*>(p.out) + int64_t(item.b) * p.num_q_heads * kD +
                                                int64_t(item.kvh * p.kv_mul + hq) * kD);
        const float inv = 1.f / L;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          __align__(16) T tmp[E];
#pragma unroll
          for (int e = 0; e < E; ++e) tmp[e] = Elt<T>::from_float(O[c * E + e] * inv);
          *reinterpret_cast<uint4*>(o + coff[c]) = *reinterpret_cast<const uint4*>(tmp);
        }
      }
      return;
    }
    // A group holds pieces of at most two such items: one that entered it from the left (0) and
    // one that starts inside it (1).
    auto group_slot = [&](int64_t g) {
      return p.partials + (group_base + 2 * g + ((c_first < g * kGroup) ? 0 : 1)) * C::kPartialFloats;
    };
    const int64_t g = worker / kGroup;
    const int64_t g_lo = c_first > g * kGroup ? c_first : g * kGroup;
    const int64_t g_hi = c_last < g * kGroup + kGroup - 1 ? c_last : g * kGroup + kGroup - 1;
    int* group_cnt = reinterpret_cast<int*>(p.partials + (int64_t(p.partial_slots) - 1) * C::kPartialFloats) +
                     2 * g + ((c_first < g * kGroup) ? 0 : 1);
    if (!arrive_last(group_cnt, int(g_hi - g_lo) + 1)) return;
    merge(g_hi - g_lo + 1, [&](int64_t i) { return slot_of(g_lo + i); }, group_slot(g));
    __syncwarp();  // every lane's part of the group slot is ordered before lane 0's release
    const int64_t G0 = c_first / kGroup, G1 = c_last / kGroup;
    if (arrive_last(item_cnt, int(G1 - G0) + 1))
      merge(G1 - G0 + 1, [&](int64_t i) { return static_cast<const float*>(group_slot(G0 + i)); }, nullptr);
  };

  auto wait_slot = [&](uint64_t* bar, uint32_t ph) -> bool {
    if (mbar_try_wait(bar, ph)) return true;
    bool ok = mbar_wait_bounded(bar, ph, p.wait_limit);
    if (!__all_sync(0xffffffffu, ok)) {
      // Give up: report, then let the tile copies this warp still has in flight land (a bounded
      // pause far longer than a copy takes) before the warp retires, so that nothing arrives in
      // shared memory that has passed to another CTA.
      if (lane == 0) atomicMax(p.status, KPX_ERR_DEVICE_TIMEOUT);
      for (int k = 0; k < 64; ++k) __nanosleep(1000);
      return false;
    }
    return true;
  };

  begin_item(n, std::true_type{});
  int64_t item_first = u0 - cur.blk;  // global block index where the current item starts
  int ks = 0, vs = 0;                 // slots of the next K block and the next V block to consume
  uint32_t kph = 0, vph = 0;          // their phase parities

  // One iteration: scores + online softmax of block i; when kPend, the output pass of
  // block i-1 sits in the same straight-line region as the shuffle chains so that its
  // loads and FMAs fill their latency.  Returns false if a bounded wait gave up.
  auto step = [&](int i, int nvalid, auto pend_tag) -> bool {
    constexpr bool kPend = decltype(pend_tag)::value;
    if (!wait_slot(bars + ks, kph)) return false;
    if (kPend) {
      if (!wait_slot(bars + NS + vs, vph)) return false;
    }
    float part[R * QH];
    {
      const uint8_t* kt = ring + ks * C::kTileB;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint8_t* krow = kt + ((r ^ perm) * TG + tg) * (kD * C::kEltB);
        float kf[DPT];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint4 raw = *reinterpret_cast<const uint4*>(krow + coff[c]);
          Elt<T>::unpack(raw, kf + c * E);
        }
#pragma unroll
        for (int j = 0; j < QH; ++j) {
          float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
          for (int d = 0; d < HP; ++d)
            s2 = __ffma2_rn(q2[j][d], make_float2(kf[2 * d], kf[2 * d + 1]), s2);
          part[r * QH + j] = s2.x + s2.y;
        }
      }
    }
    // halving over the row index: the upper half of the registers goes to lane ^ (LPT/2), then
    // lane ^ (LPT/4), ... down to lane ^ 2; what is left is token row perm*TG + tg
#pragma unroll
    for (int m = LPT / 2, half = R * QH / 2; m >= 2; m >>= 1, half >>= 1) {
#pragma unroll
      for (int k = 0; k < R * QH / 2; ++k)
        if (k < half) part[k] += __shfl_xor_sync(0xffffffffu, part[half + k], m);
    }
    if (QH == 4) {
      float s0 = hi_lane ? part[0] : part[2], s1 = hi_lane ? part[1] : part[3];
      float k0 = hi_lane ? part[2] : part[0], k1 = hi_lane ? part[3] : part[1];
      part[0] = k0 + __shfl_xor_sync(0xffffffffu, s0, 1);
      part[1] = k1 + __shfl_xor_sync(0xffffffffu, s1, 1);
    } else if (QH == 2) {
      float s0 = hi_lane ? part[0] : part[1], k0 = hi_lane ? part[1] : part[0];
      part[0] = k0 + __shfl_xor_sync(0xffffffffu, s0, 1);
    } else {
      part[0] += __shfl_xor_sync(0xffffffffu, part[0], 1);
    }
    const bool tok_ok = (perm * TG + tg) < nvalid;
    float alpha[NV];
    bool changed = false;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float sc = tok_ok ? part[k] : -INFINITY;
      float mx = sc;
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m_run[k], mx);
      alpha[k] = fast_exp2(m_run[k] - m_new);
      changed |= (m_new != m_run[k]);
      m_run[k] = m_new;
      const float pw = fast_exp2(sc - m_new);
      l_run[k] = l_run[k] * alpha[k] + pw;
      part[k] = pw;
    }
    if (kPend)
      pv_pass(ring + (NS + vs) * C::kTileB, p_s + ((i - 1) & 1) * (kBS * 4), kBS, std::true_type{});
    float* pb_new = p_s + (i & 1) * (kBS * 4);
    if (QH == 4) {
      *reinterpret_cast<float2*>(pb_new + (perm * TG + tg) * 4 + my_j0) = make_float2(part[0], part[1]);
    } else {
      pb_new[(perm * TG + tg) * 4 + my_j0] = part[0];
    }
    if (__any_sync(0xffffffffu, changed)) {
      float al[QH];
      if (QH == 4) {
        float o0 = __shfl_xor_sync(0xffffffffu, alpha[0], 1);
        float o1 = __shfl_xor_sync(0xffffffffu, alpha[NV - 1], 1);
        al[0] = hi_lane ? o0 : alpha[0];
        al[1 % QH] = hi_lane ? o1 : alpha[NV - 1];
        al[2 % QH] = hi_lane ? alpha[0] : o0;
        al[3 % QH] = hi_lane ? alpha[NV - 1] : o1;
      } else if (QH == 2) {
        float o0 = __shfl_xor_sync(0xffffffffu, alpha[0], 1);
        al[0] = hi_lane ? o0 : alpha[0];
        al[1 % QH] = hi_lane ? alpha[0] : o0;
      } else {
        al[0] = alpha[0];
      }
#pragma unroll
      for (int j = 0; j < QH; ++j)
#pragma unroll
        for (int d = 0; d < HP; ++d) {
          acc[j][d].x *= al[j];
          acc[j][d].y *= al[j];
        }
    }
    __syncwarp();  // K(i) and V(i-1) fully read; p(i) visible to the whole warp
    // ---------------- refill the slots just left ----------------
    if (lane == 0) fence_proxy_async();
    if (kPend) {
      if (v_issued < n) issue_v(vs);
      if (++vs == NS) { vs = 0; vph ^= 1; }
    }
    if (k_issued < n) issue_k(ks);
    if (++ks == NS) { ks = 0; kph ^= 1; }
    return true;
  };

  // The range is a sequence of segments, each the part of one item that falls in it.
  int i = 0;
  while (i < n) {
    const int m = min(n - i, cur.nblk - cur.blk);           // blocks of this item in the range
    if (i + m < n && lane < QH * 2) {
      // the next segment starts a new item: pull its query rows towards L2 now (128-byte lines)
      Cursor nx = cur;
      nx.blk += m - 1;
      nx.advance(p, prefix);
      const int hgn = nx.sub - nx.kvh * p.head_groups;
      const int hqn = min(hgn * QH + (lane >> 1), p.kv_mul - 1);
      const uint8_t* qn = static_cast<const uint8_t*>(p.q) +
                          (int64_t(nx.b) * p.num_q_heads + nx.kvh * p.kv_mul + hqn) * (kD * C::kEltB) +
                          (lane & 1) * (kD * C::kEltB / 2);
      asm volatile("prefetch.global.L2 [%0];" ::"l"(qn));
    }
    if constexpr (kFused) {
      if (i + m < n && lane >= 8 && lane < 20) {
        // ... and the rows the fused step rotates with: the new token's K and V rows (two
        // 128-byte lines each for 16-bit elements) and the sin / cos rows of its position
        Cursor nx = cur;
        nx.blk += m - 1;
        nx.advance(p, prefix);
        const int64_t kv_row = (int64_t(nx.b) * p.num_kv_heads + nx.kvh) * (kD * C::kEltB);
        const int l = lane - 8;
        const uint8_t* src =
            l < 2   ? static_cast<const uint8_t*>(p.k_new) + kv_row + l * (kD * C::kEltB / 2)
            : l < 4 ? static_cast<const uint8_t*>(p.v_new) + kv_row + (l - 2) * (kD * C::kEltB / 2)
            : l < 8 ? reinterpret_cast<const uint8_t*>(p.sin_cache + int64_t(nx.len) * kD) + (l - 4) * 128
                    : reinterpret_cast<const uint8_t*>(p.cos_cache + int64_t(nx.len) * kD) + (l - 8) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
      }
    }
    const bool to_item_end = (cur.blk + m == cur.nblk);
    const int tail_valid = to_item_end ? cur.len - (cur.nblk - 1) * kBS : kBS;  // tokens in the segment's last block
    if (!step(i, m == 1 ? tail_valid : kBS, std::false_type{})) return;
    for (int t = 1; t < m; ++t)
      if (!step(i + t, t == m - 1 ? tail_valid : kBS, std::true_type{})) return;
    i += m;
    // flush: output pass of the segment's last block (possibly a partial block)
    if (!wait_slot(bars + NS + vs, vph)) return;
    pv_pass(ring + (NS + vs) * C::kTileB, p_s + ((i - 1) & 1) * (kBS * 4), tail_valid, std::false_type{});
    __syncwarp();
    if (lane == 0) fence_proxy_async();
    if (v_issued < n) issue_v(vs);
    if (++vs == NS) { vs = 0; vph ^= 1; }
    const int64_t item_end = item_first + cur.nblk;
    const bool whole = (item_first >= u0) && (item_end <= u1);
    const int64_t pslot = (item_first < u0) ? 2 * worker : 2 * worker + 1;
    end_item(cur, whole, pslot, item_first, to_item_end);
    if (i < n) {
      cur.blk += m - 1;
      cur.advance(p, prefix);
      item_first = item_end;
      begin_item(n - i, std::false_type{});
    }
  }
}

inline int heads_per_warp(int kv_mul);
inline int64_t counter_bytes(int num_q_heads, int num_kv_heads) {
  const int kv_mul = num_q_heads / num_kv_heads;
  const int qh = heads_per_warp(kv_mul);
  const int64_t items = int64_t(kMaxBatch) * num_kv_heads * ((kv_mul + qh - 1) / qh);
  return (items * 4 + 255) / 256 * 256;
}
inline int heads_per_warp(int kv_mul) {
  if (kv_mul == 1) return 1;
  if (kv_mul == 2) return 2;
  return 4;
}

constexpr int kMaxSms = 160;  // upper bound used to size the workspace
constexpr int kMaxWarpsPerCta = 16;
constexpr int kMinPartialSlots = 2 * kMaxSms * kMaxWarpsPerCta;  // two per warp of the largest grid
constexpr int kStatusBytes = 256;

// Tuning knob: 0 = default shape; set through kpx_internal_set_decode_variant.
extern int g_decode_variant;
// Small launches (see paged_decode_kernel): used when batch x table width x items per sequence
// is below g_small_below blocks per warp of the grid; then ranges hold at least
// g_min_blocks_per_range blocks while at least g_min_warps_per_sm warps per SM stay active.
extern int g_small_below, g_min_blocks_per_range, g_min_warps_per_sm;
extern uint32_t g_wait_limit;
extern int g_withhold_worker;

// True when the launch certainly has fewer than g_small_below blocks per warp.  What bounds a
// sequence's blocks on the host: the table width; without a table (the reference's contiguous
// cache) the fixed length if there is one, else the cache's size if the layout states it.
inline bool small_launch(const DecodeParams& p, int qh, int warps_per_cta) {
  if (g_small_below <= 0) return false;
  int64_t per_seq_blocks;
  if (p.block_table) per_seq_blocks = p.max_blocks_per_seq;
  else if (!p.seq_lens) per_seq_blocks = (int64_t(p.len_bias) + kBS - 1) / kBS;
  else if (p.num_blocks > 0) per_seq_blocks = p.num_blocks;
  else return false;
  int grid = device_info().sm_count;
  if (grid > kMaxSms) grid = kMaxSms;
  const int64_t groups = (p.kv_mul + qh - 1) / qh;
  const int64_t bound = int64_t(p.batch) * per_seq_blocks * p.num_kv_heads * groups;
  return bound < int64_t(grid) * warps_per_cta * g_small_below;
}

template <typename T, int QH, int NW, int NS, int LPT, bool kSmall, int CPS, bool kFused>
int launch_decode_form(DecodeParams p, cudaStream_t stream) {
  using C = Cfg<T, QH, NW, NS, LPT>;
  // the shared-memory attribute is set once per device and kernel form; the bit mask makes
  // concurrent first calls and processes that alternate devices safe
  constexpr int smem_bytes = kFused ? C::kSmemFused : C::kSmem;
  static std::atomic<uint64_t> configured{0};
  int dev = 0;
  KPX_CUDA_TRY(cudaGetDevice(&dev));
  auto kern = paged_decode_kernel<T, QH, NW, NS, LPT, kSmall, CPS, kFused>;
  const uint64_t bit = uint64_t(1) << (dev & 63);
  if (dev >= 64 || !(configured.load(std::memory_order_acquire) & bit)) {
    KPX_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    if (dev < 64) configured.fetch_or(bit, std::memory_order_release);
  }
  int grid = device_info().sm_count;
  if (grid > kMaxSms) grid = kMaxSms;
  grid *= CPS;
  p.head_groups = (p.kv_mul + QH - 1) / QH;
  kern<<<grid, C::kThreads, smem_bytes, stream>>>(p);
  KPX_CUDA_TRY(cudaGetLastError());
  return cuda_status(cudaGetLastError());
}

template <typename T, int QH, int NW, int NS, int LPT, bool kSmall = false, int CPS = 1>
int launch_decode(const DecodeParams& p, cudaStream_t stream) {
  return p.k_new ? launch_decode_form<T, QH, NW, NS, LPT, kSmall, CPS, true>(p, stream)
                 : launch_decode_form<T, QH, NW, NS, LPT, kSmall, CPS, false>(p, stream);
}

template <typename T, int QH>
int launch_shape(const DecodeParams& p, cudaStream_t stream, int flags) {
  // Launches that the caller overlaps on the GPU (KPX_DECODE_OVERLAPPED) run as three small CTAs
  // per SM instead of one large one: an SM then takes up the next launch's work a third at a
  // time while the previous launch's last warps finish.  Alone, the large CTA is faster.
  const bool overlapped = (flags & KPX_DECODE_OVERLAPPED) != 0;
  if (sizeof(T) == 4) {
    if (small_launch(p, QH, 6)) return launch_decode<T, QH, 6, 2, 8, true>(p, stream);
    return overlapped ? launch_decode<T, QH, 2, 2, 8, false, 3>(p, stream)
                      : launch_decode<T, QH, 6, 2, 8>(p, stream);
  }
  // tuning knob for experiments: 1 forces the three-small-CTAs form, 2 the one-large-CTA form
  const bool small_ctas = (g_decode_variant & 3) == 1 ? true : ((g_decode_variant & 3) == 2 ? false : overlapped);
  if (small_launch(p, QH, 12)) return launch_decode<T, QH, 12, 2, 16, true>(p, stream);
  return small_ctas ? launch_decode<T, QH, 4, 2, 16, false, 3>(p, stream)
                    : launch_decode<T, QH, 12, 2, 16>(p, stream);
}

#ifdef KPX_DECODE_INSTANTIATE
template <typename T>
int dispatch_decode(const DecodeParams& p, cudaStream_t stream, int flags) {
  switch (heads_per_warp(p.kv_mul)) {
    case 1: return launch_shape<T, 1>(p, stream, flags);
    case 2: return launch_shape<T, 2>(p, stream, flags);
    default: return launch_shape<T, 4>(p, stream, flags);
  }
}

#else
template <typename T>
int dispatch_decode(const DecodeParams& p, cudaStream_t stream, int flags);
#endif

}  // namespace decode
}  // namespace kpx
