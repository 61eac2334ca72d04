// Paged GQA decode attention for sm_100a: persistent split-KV kernel + merge.
//
// Work decomposition.  The cache of sequence b holds len_b tokens in blocks of 16;
// a "stage unit" is 4 consecutive blocks (64 tokens) of one (sequence, kv head)
// item.  All stage units of all items are laid on one line (sequence-major, kv
// head next) and cut into G equal contiguous ranges, one per persistent CTA
// (G = resident CTAs on the GPU), so every CTA streams the same number of bytes
// whatever the spread of sequence lengths.  A CTA that covers an item completely
// writes its output directly; an item cut by a range boundary leaves one partial
// (running max, sum, un-normalised accumulator) per CTA in the workspace and a
// small second kernel merges them.
//
// Inside a CTA, K/V tiles are gathered through the block table with cp.async.bulk
// (the TMA engine) into a ring of shared-memory stages guarded by full/empty
// mbarriers; warp 0 issues the copies for the stage kStages ahead right after it
// has finished its share of the current one (a dedicated producer warp would push
// one scheduler to 3 warps and cap every thread at 168 registers).  4 warps per
// group of up to 4 query heads each take one block of the stage, so a K/V byte is
// fetched from HBM once for all query heads that share the KV head.  The math is
// fp32 on CUDA cores (packed fp32x2 FMAs), softmax is online with warp shuffles.
// Every mbarrier wait is bounded; a wait that gives up raises the workspace status
// word and the CTA drains without touching shared data again.
#include "kpx_common.cuh"

namespace kpx {
namespace {

constexpr int kD = 128;       // head size
constexpr int kBS = 16;       // tokens per block
constexpr int kBPS = 4;       // blocks per stage (= consumer warps per head group)
constexpr int kMaxBatch = 1024;  // sequences per launch (prefix table lives in smem)
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeParams {
  void* out;
  const void* q;
  const uint8_t* k_pool;
  const uint8_t* v_pool;
  const int32_t* block_table;
  const int32_t* seq_lens;
  float* partials;
  int32_t* status;
  int64_t block_stride_b, head_stride_b, token_stride_b;  // bytes
  int64_t num_blocks;
  int32_t max_blocks_per_seq, len_bias, batch;
  int32_t num_q_heads, num_kv_heads, kv_mul;
  int32_t tile_contig;
  float qscale;  // softmax scale * log2(e)
};

template <typename T, int QH, int HG>
struct Cfg {
  static constexpr int kEltB = sizeof(T);
  static constexpr int kTileB = kBS * kD * kEltB;               // one (block, head) tile
  static constexpr int kStageB = 2 * kBPS * kTileB;             // K then V
  static constexpr int kStages = (kEltB == 2) ? (HG == 1 ? 3 : 5) : (HG == 1 ? 3 : 3);
  static constexpr int kConsumerWarps = kBPS * HG;
  static constexpr int kThreads = 32 * kConsumerWarps;
  static constexpr int kCtasPerSm = (kEltB == 2 && HG == 1) ? 2 : 1;
  // shared memory carve-up (bytes)
  static constexpr int kOffBars = kStages * kStageB;
  static constexpr int kOffPrefix = kOffBars + 2 * kStages * 8 + 16;
  static constexpr int kOffP = kOffPrefix + (kMaxBatch + 1) * 4 + 12;
  static constexpr int kOffMerge = kOffP + kConsumerWarps * kBS * 4 * 4;
  static constexpr int kMergeFloats = kBPS * QH * (kD + 2);  // per head group
  static constexpr int kSmem = kOffMerge + HG * kMergeFloats * 4;
  static constexpr int kPartialFloats = HG * QH * (kD + 2);  // one workspace slot
};

__device__ __forceinline__ int seq_len_of(const DecodeParams& p, int b) {
  int len = (p.seq_lens ? p.seq_lens[b] : 0) + p.len_bias;
  return len < 0 ? 0 : len;
}

// Walks the stage units of a CTA's range in order.
struct Cursor {
  int b, kvh, off, su, len;
  __device__ __forceinline__ void locate(const DecodeParams& p, const int* prefix, int64_t u) {
    // first i with Hkv*prefix[i] > u, then b = i-1
    int lo = 0, hi = p.batch;
    while (lo < hi) {
      int mid = (lo + hi) >> 1;
      if (int64_t(prefix[mid + 1]) * p.num_kv_heads > u) hi = mid; else lo = mid + 1;
    }
    b = lo;
    su = prefix[b + 1] - prefix[b];
    int64_t r = u - int64_t(prefix[b]) * p.num_kv_heads;
    kvh = int(r / su);
    off = int(r - int64_t(kvh) * su);
    len = seq_len_of(p, b);
  }
  // returns true when the step left the current item
  __device__ __forceinline__ bool advance(const DecodeParams& p, const int* prefix) {
    if (++off < su) return false;
    off = 0;
    if (++kvh == p.num_kv_heads) {
      kvh = 0;
      do { ++b; } while (b < p.batch && prefix[b + 1] == prefix[b]);
      if (b < p.batch) {
        su = prefix[b + 1] - prefix[b];
        len = seq_len_of(p, b);
      }
    }
    return true;
  }
};

__device__ __forceinline__ int64_t range_start(int64_t total, int c, int g) {
  return (total * c) / g;
}

// Sum-reduce N per-thread partials across the 8 lanes of a token group by
// recursive halving: after the step with lane mask m a lane keeps the lower half
// of its values if (sub & m) == 0, the upper half otherwise.  Leaves max(1, N/8)
// finished values in v[0..].
template <int N>
__device__ __forceinline__ void reduce_scatter8(float* v, int sub) {
  int n = N;
#pragma unroll
  for (int m = 4; m >= 1; m >>= 1) {
    if (n >= 2) {
      const int half = n / 2;
      const bool upper = (sub & m) != 0;
#pragma unroll
      for (int i = 0; i < N / 2; ++i) {
        if (i < half) {
          float send = upper ? v[i] : v[i + half];
          float keep = upper ? v[i + half] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, m);
        }
      }
      n = half;
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], m);
    }
  }
}

template <typename T, int QH, int HG>
__global__ void __launch_bounds__(Cfg<T, QH, HG>::kThreads, Cfg<T, QH, HG>::kCtasPerSm)
paged_decode_kernel(const DecodeParams p) {
  using C = Cfg<T, QH, HG>;
  constexpr int E = Elt<T>::kPer16B;      // elements per 16-byte vector
  constexpr int NCH = 16 / E;             // 16-byte chunks per thread per row (16 dims)
  constexpr int NV = (4 * QH >= 8) ? (4 * QH / 8) : 1;  // finished scores per thread per block
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kOffBars);
  uint64_t* empty_bar = full_bar + C::kStages;
  int* prefix = reinterpret_cast<int*>(smem + C::kOffPrefix);
  int* abort_flag = prefix + kMaxBatch + 1;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;

  // ---- set-up: stage-unit prefix over sequences, barriers ----
  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, C::kConsumerWarps);
    }
    mbar_fence_init();
    *abort_flag = 0;
  }
  for (int b = tid; b < p.batch; b += C::kThreads) {
    int len = seq_len_of(p, b);
    prefix[b + 1] = (len + kBS * kBPS - 1) / (kBS * kBPS);
  }
  if (tid == 0) prefix[0] = 0;
  __syncthreads();
  if (warp == 0) {  // inclusive scan, one warp, chunks of 32
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
  const int64_t total_units = int64_t(prefix[p.batch]) * p.num_kv_heads;
  const int64_t u0 = range_start(total_units, cta, G), u1 = range_start(total_units, cta + 1, G);
  if (u0 >= u1) return;
  const int n_units = int(u1 - u0);

  // ============================ producer role (warp 0) ============================
  // Warp 0 doubles as the producer: after it has finished a stage it refills that
  // slot with the unit kStages ahead.  Lanes 0..3 fetch the block ids of a unit one
  // iteration before they are needed, so the table lookup is off the critical path.
  Cursor pcur;            // next unit to issue
  int p_next_id = -1;     // block id (lanes 0..3) of the unit at pcur
  int p_issued = 0;       // units issued so far
  auto load_id = [&](const Cursor& c) -> int {
    int blk = c.off * kBPS + (lane & 3);
    int nblk = (c.len + kBS - 1) / kBS;
    if (lane >= kBPS || blk >= nblk) return -1;
    int id = p.block_table ? p.block_table[int64_t(c.b) * p.max_blocks_per_seq + blk] : blk;
    if (id < 0 || (p.num_blocks > 0 && id >= p.num_blocks)) {
      atomicMax(p.status, KPX_ERR_INVALID_ARGUMENT);
      id = 0;
    }
    return id;
  };
  // issue the copies of the unit at pcur into `slot` (the slot must be free), then
  // step pcur and prefetch the ids of the following unit
  auto issue_next = [&]() {
    const int slot = p_issued % C::kStages;
    const Cursor here = pcur;
    const int my_id = p_next_id;
    const int nblk = (here.len + kBS - 1) / kBS;
    const int nb = min(kBPS, nblk - here.off * kBPS);
    uint8_t* stage = smem + slot * C::kStageB;
    if (p.tile_contig) {
      if (lane == 0) mbar_arrive_expect_tx(full_bar + slot, uint32_t(nb) * 2u * C::kTileB);
      __syncwarp();
      int blk = lane >> 1, which = lane & 1;  // lane -> (block, K/V)
      int id = __shfl_sync(0xffffffffu, my_id, blk & 3);
      if (lane < 2 * nb) {
        const uint8_t* src = (which ? p.v_pool : p.k_pool) + int64_t(id) * p.block_stride_b +
                             int64_t(here.kvh) * p.head_stride_b;
        bulk_g2s(stage + which * (kBPS * C::kTileB) + blk * C::kTileB, src, C::kTileB,
                 full_bar + slot);
      }
    } else {
      // strided rows (the reference's token-major cache): one bulk copy per valid row
      constexpr int kRowB = kD * C::kEltB;
      int rows_total = min(here.len - here.off * kBPS * kBS, kBPS * kBS);
      if (lane == 0) mbar_arrive_expect_tx(full_bar + slot, uint32_t(rows_total) * 2u * kRowB);
      __syncwarp();
      for (int c = lane; c < 2 * kBPS * kBS; c += 32) {
        int blk = c >> 5, which = (c >> 4) & 1, row = c & 15;
        int id = __shfl_sync(0xffffffffu, my_id, blk);
        if (blk * kBS + row < rows_total) {
          const uint8_t* src = (which ? p.v_pool : p.k_pool) + int64_t(id) * p.block_stride_b +
                               int64_t(here.kvh) * p.head_stride_b + int64_t(row) * p.token_stride_b;
          bulk_g2s(stage + which * (kBPS * C::kTileB) + blk * C::kTileB + row * kRowB, src, kRowB,
                   full_bar + slot);
        }
      }
    }
    ++p_issued;
    pcur.advance(p, prefix);
    if (p_issued < n_units) p_next_id = load_id(pcur);
  };
  if (warp == 0) {
    pcur.locate(p, prefix, u0);
    p_next_id = load_id(pcur);
    const int pre = min(n_units, C::kStages);
    for (int i = 0; i < pre; ++i) issue_next();
  }

  // ================================ consumer warps =================================
  const int hg = warp / kBPS;     // head group of this warp
  const int wb = warp % kBPS;     // block of the stage this warp owns
  const int tg = lane >> 3;       // token group 0..3: tokens it*4+tg
  const int sub = lane & 7;       // 16 of the 128 dims
  float* p_s = reinterpret_cast<float*>(smem + C::kOffP) + warp * (kBS * 4);
  float* mg = reinterpret_cast<float*>(smem + C::kOffMerge) + hg * C::kMergeFloats;
  float* mg_acc = mg;                       // [kBPS][QH][kD]
  float* mg_m = mg + kBPS * QH * kD;        // [kBPS][QH]
  float* mg_l = mg_m + kBPS * QH;           // [kBPS][QH]
  const int gtid = tid - hg * (32 * kBPS);  // 0..127 inside the head group
  const int bar_id = 1 + hg;

  // element offset of this thread's chunk c inside a 128-wide row
  auto chunk_off = [&](int c) -> int { return c * (kD / NCH) + sub * E; };

  // which finished scores this thread ends up with after reduce_scatter8
  int my_it, my_j0;
  if (QH == 4) { my_it = ((sub >> 2) & 1) * 2 + ((sub >> 1) & 1); my_j0 = (sub & 1) * 2; }
  else if (QH == 2) { my_it = sub >> 1; my_j0 = sub & 1; }
  else { my_it = sub >> 1; my_j0 = 0; }

  Cursor cur;
  cur.locate(p, prefix, u0);
  bool aborted = false;

  float2 q2[QH][8];
  float2 acc[QH][8];
  float m_run[NV], l_run[NV];

  auto begin_item = [&]() {
    const T* qrow = static_cast<const T*>(p.q) + int64_t(cur.b) * p.num_q_heads * kD;
#pragma unroll
    for (int j = 0; j < QH; ++j) {
      int hq = hg * QH + j;
      bool valid = hq < p.kv_mul;
      const T* qh = qrow + int64_t(cur.kvh * p.kv_mul + (valid ? hq : 0)) * kD;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        float f[E];
        uint4 raw = __ldg(reinterpret_cast<const uint4*>(qh + chunk_off(c)));
        Elt<T>::unpack(raw, f);
#pragma unroll
        for (int e = 0; e < E; e += 2) {
          float sc = valid ? p.qscale : 0.f;
          q2[j][(c * E + e) / 2] = make_float2(f[e] * sc, f[e + 1] * sc);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[j][i] = make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) { m_run[k] = -INFINITY; l_run[k] = 0.f; }
  };

  auto end_item = [&](const Cursor& item, bool whole_item, int partial_slot) {
    // reduce over the 4 token groups of the warp
#pragma unroll
    for (int j = 0; j < QH; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float2 a = acc[j][i];
        a.x += __shfl_xor_sync(0xffffffffu, a.x, 8);
        a.y += __shfl_xor_sync(0xffffffffu, a.y, 8);
        a.x += __shfl_xor_sync(0xffffffffu, a.x, 16);
        a.y += __shfl_xor_sync(0xffffffffu, a.y, 16);
        acc[j][i] = a;
      }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float l = l_run[k];
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      l_run[k] = l;
    }
    if (tg == 0) {
#pragma unroll
      for (int j = 0; j < QH; ++j)
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
          for (int e = 0; e < E; e += 2) {
            float2 a = acc[j][(c * E + e) / 2];
            *reinterpret_cast<float2*>(mg_acc + (wb * QH + j) * kD + chunk_off(c) + e) = a;
          }
      // one lane per finished-score owner publishes m and l of its heads
      bool owner = (QH == 4) ? (sub < 2) : (QH == 2 ? (sub < 2) : (sub == 0));
      if (owner) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          mg_m[wb * QH + my_j0 + k] = m_run[k];
          mg_l[wb * QH + my_j0 + k] = l_run[k];
        }
      }
    }
    named_bar_sync(bar_id, 32 * kBPS);
    // combine the 4 warps: thread gtid owns dim gtid of every head
    T* orow = static_cast<T*>(p.out) + int64_t(item.b) * p.num_q_heads * kD;
    float* pslot = p.partials + int64_t(partial_slot) * C::kPartialFloats;
#pragma unroll
    for (int j = 0; j < QH; ++j) {
      int hq = hg * QH + j;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kBPS; ++w) M = fmaxf(M, mg_m[w * QH + j]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < kBPS; ++w) {
        float mw = mg_m[w * QH + j];
        float sc = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
        L += mg_l[w * QH + j] * sc;
        O += mg_acc[(w * QH + j) * kD + gtid] * sc;
      }
      if (hq < p.kv_mul) {
        if (whole_item) {
          orow[int64_t(item.kvh * p.kv_mul + hq) * kD + gtid] = Elt<T>::from_float(O / L);
        } else {
          pslot[hq * kD + gtid] = O;
          if (gtid == 0) {
            pslot[HG * QH * kD + hq] = M;
            pslot[HG * QH * kD + HG * QH + hq] = L;
          }
        }
      }
    }
    named_bar_sync(bar_id, 32 * kBPS);
  };

  begin_item();
  int64_t item_first_unit = u0 - cur.off;  // global unit index where the current item starts
  for (int it = 0; it < n_units; ++it) {
    const int slot = it % C::kStages;
    if (!aborted) {
      if (!mbar_wait_bounded(full_bar + slot, (it / C::kStages) & 1)) {
        aborted = true;
        *reinterpret_cast<volatile int*>(abort_flag) = 1;
        atomicMax(p.status, KPX_ERR_DEVICE_TIMEOUT);
      }
    }
    aborted = __any_sync(0xffffffffu, aborted || *reinterpret_cast<volatile int*>(abort_flag) != 0);
    const int blk = cur.off * kBPS + wb;
    const int nvalid = cur.len - blk * kBS;  // tokens of this block that exist (may be <= 0)
    if (!aborted && nvalid > 0) {
      const uint8_t* kt = smem + slot * C::kStageB + wb * C::kTileB;
      const uint8_t* vt = kt + kBPS * C::kTileB;
      // ---- scores: s[it][j] partial over this thread's 16 dims ----
      float part[4 * QH];
#pragma unroll
      for (int i4 = 0; i4 < 4; ++i4) {
        const int tok = i4 * 4 + tg;
        float kf[16];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint4 raw = *reinterpret_cast<const uint4*>(kt + (tok * kD + chunk_off(c)) * C::kEltB);
          Elt<T>::unpack(raw, kf + c * E);
        }
#pragma unroll
        for (int j = 0; j < QH; ++j) {
          float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            s2 = __ffma2_rn(q2[j][i], make_float2(kf[2 * i], kf[2 * i + 1]), s2);
          part[i4 * QH + j] = s2.x + s2.y;
        }
      }
      reduce_scatter8<4 * QH>(part, sub);
      // ---- online softmax on this thread's NV finished scores (token my_it*4+tg) ----
      const bool tok_ok = (my_it * 4 + tg) < nvalid;
      float alpha[NV];
      bool changed = false;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        float s = tok_ok ? part[k] : -INFINITY;
        float mx = s;
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        float m_new = fmaxf(m_run[k], mx);
        alpha[k] = fast_exp2(m_run[k] - m_new);
        changed |= (m_new != m_run[k]);
        m_run[k] = m_new;
        float pv = fast_exp2(s - m_new);
        l_run[k] = l_run[k] * alpha[k] + pv;
        part[k] = pv;
      }
      if (QH == 4) {
        *reinterpret_cast<float2*>(p_s + (my_it * 4 + tg) * 4 + my_j0) = make_float2(part[0], part[1]);
      } else {
        p_s[(my_it * 4 + tg) * 4 + my_j0] = part[0];
      }
      if (__any_sync(0xffffffffu, changed)) {
        // rescale the accumulators of every head; fetch the other lanes' factors
        float al[QH];
        if (QH == 4) {
          float o0 = __shfl_xor_sync(0xffffffffu, alpha[0], 1);
          float o1 = __shfl_xor_sync(0xffffffffu, alpha[NV - 1], 1);
          bool hi = (sub & 1) != 0;
          al[0] = hi ? o0 : alpha[0];
          al[1] = hi ? o1 : alpha[NV - 1];
          al[2 % QH] = hi ? alpha[0] : o0;
          al[3 % QH] = hi ? alpha[NV - 1] : o1;
        } else if (QH == 2) {
          float o0 = __shfl_xor_sync(0xffffffffu, alpha[0], 1);
          bool hi = (sub & 1) != 0;
          al[0] = hi ? o0 : alpha[0];
          al[1 % QH] = hi ? alpha[0] : o0;
        } else {
          al[0] = alpha[0];
        }
#pragma unroll
        for (int j = 0; j < QH; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            acc[j][i].x *= al[j];
            acc[j][i].y *= al[j];
          }
      }
      __syncwarp();
      // ---- out += p * V ----
#pragma unroll
      for (int i4 = 0; i4 < 4; ++i4) {
        const int tok = i4 * 4 + tg;
        if (tok < nvalid) {
          float vf[16];
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            uint4 raw = *reinterpret_cast<const uint4*>(vt + (tok * kD + chunk_off(c)) * C::kEltB);
            Elt<T>::unpack(raw, vf + c * E);
          }
          float pj[4];
          if (QH == 4) {
            float4 t4 = *reinterpret_cast<const float4*>(p_s + tok * 4);
            pj[0] = t4.x; pj[1] = t4.y; pj[2] = t4.z; pj[3] = t4.w;
          } else if (QH == 2) {
            float2 t2 = *reinterpret_cast<const float2*>(p_s + tok * 4);
            pj[0] = t2.x; pj[1] = t2.y;
          } else {
            pj[0] = p_s[tok * 4];
          }
#pragma unroll
          for (int j = 0; j < QH; ++j) {
            float2 pp = make_float2(pj[j], pj[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              acc[j][i] = __ffma2_rn(pp, make_float2(vf[2 * i], vf[2 * i + 1]), acc[j][i]);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar + slot);
    if (warp == 0 && p_issued < n_units) {
      // refill this slot once all consumer warps have released it
      if (!aborted && !mbar_wait_bounded(empty_bar + slot, (it / C::kStages) & 1)) {
        aborted = true;
        *reinterpret_cast<volatile int*>(abort_flag) = 1;
        atomicMax(p.status, KPX_ERR_DEVICE_TIMEOUT);
      }
      aborted = __any_sync(0xffffffffu, aborted);
      if (!aborted) issue_next();
    }

    const Cursor item = cur;
    const bool left = cur.advance(p, prefix);
    const bool last = (it + 1 == n_units);
    if (left || last) {
      const int64_t item_end = item_first_unit + item.su;
      const bool whole = (item_first_unit >= u0) && (item_end <= u1);
      const int pslot = (item_first_unit < u0) ? 2 * cta : 2 * cta + 1;
      end_item(item, whole, pslot);
      if (!last) {
        item_first_unit = item_end;
        begin_item();
      }
    }
  }
}

// Second pass: items cut by a CTA range boundary are assembled from the partials
// of the CTAs that touched them; empty sequences get zeros.  One CTA per
// (sequence, kv head), one thread per output dim.
template <typename T>
__global__ void __launch_bounds__(kD) decode_merge_kernel(const DecodeParams p, int G, int slot_floats,
                                                          int hq_total) {
  __shared__ int s_prefix_b, s_su;
  const int item = blockIdx.x;
  const int b = item / p.num_kv_heads, kvh = item - b * p.num_kv_heads;
  const int tid = threadIdx.x;
  // stage-unit prefix of this sequence (batch is small: a serial scan by one warp is enough)
  if (tid < 32) {
    int64_t acc = 0, tot = 0;
    for (int base = 0; base < p.batch; base += 32) {
      int i = base + tid;
      int su = 0;
      if (i < p.batch) su = (seq_len_of(p, i) + kBS * kBPS - 1) / (kBS * kBPS);
      int before = (i < b) ? su : 0;
#pragma unroll
      for (int d = 16; d >= 1; d >>= 1) {
        before += __shfl_xor_sync(0xffffffffu, before, d);
        su += __shfl_xor_sync(0xffffffffu, su, d);
      }
      acc += before;
      tot += su;
    }
    if (tid == 0) {
      s_prefix_b = int(acc);
      s_su = int(tot);
    }
  }
  __syncthreads();
  const int su_b = (seq_len_of(p, b) + kBS * kBPS - 1) / (kBS * kBPS);
  T* orow = static_cast<T*>(p.out) + int64_t(b) * p.num_q_heads * kD + int64_t(kvh) * p.kv_mul * kD;
  if (su_b == 0) {
    for (int h = 0; h < p.kv_mul; ++h) orow[h * kD + tid] = Elt<T>::from_float(0.f);
    return;
  }
  const int64_t total = int64_t(s_su) * p.num_kv_heads;
  const int64_t s_i = int64_t(s_prefix_b) * p.num_kv_heads + int64_t(kvh) * su_b;
  const int64_t e_i = s_i + su_b;
  auto owner_of = [&](int64_t u) -> int {
    int c = int((u * G) / total);
    if (c >= G) c = G - 1;
    while (c + 1 < G && range_start(total, c + 1, G) <= u) ++c;
    while (c > 0 && range_start(total, c, G) > u) --c;
    return c;
  };
  const int c_first = owner_of(s_i), c_last = owner_of(e_i - 1);
  if (c_first == c_last) return;  // written directly by its only CTA
  for (int h = 0; h < p.kv_mul; ++h) {
    float M = -INFINITY;
    for (int c = c_first; c <= c_last; ++c) {
      if (range_start(total, c, G) >= range_start(total, c + 1, G)) continue;  // CTA had no units
      int slot = (s_i < range_start(total, c, G)) ? 2 * c : 2 * c + 1;
      M = fmaxf(M, p.partials[int64_t(slot) * slot_floats + hq_total * kD + h]);
    }
    float L = 0.f, O = 0.f;
    for (int c = c_first; c <= c_last; ++c) {
      if (range_start(total, c, G) >= range_start(total, c + 1, G)) continue;
      int slot = (s_i < range_start(total, c, G)) ? 2 * c : 2 * c + 1;
      const float* ps = p.partials + int64_t(slot) * slot_floats;
      float mw = ps[hq_total * kD + h];
      float sc = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
      L += ps[hq_total * kD + hq_total + h] * sc;
      O += ps[h * kD + tid] * sc;
    }
    orow[h * kD + tid] = Elt<T>::from_float(O / L);
  }
}

struct DecodePlan {
  int qh = 0, hg = 0;
};
inline bool plan_for(int kv_mul, DecodePlan* pl) {
  if (kv_mul < 1 || kv_mul > 8) return false;
  if (kv_mul == 1) { pl->qh = 1; pl->hg = 1; }
  else if (kv_mul == 2) { pl->qh = 2; pl->hg = 1; }
  else if (kv_mul <= 4) { pl->qh = 4; pl->hg = 1; }
  else { pl->qh = 4; pl->hg = 2; }
  return true;
}

constexpr int kMaxGrid = 148 * 2 * 2;  // upper bound used to size the workspace
constexpr int kStatusBytes = 256;

template <typename T, int QH, int HG>
int launch_decode(const DecodeParams& p, cudaStream_t stream, int* grid_out) {
  using C = Cfg<T, QH, HG>;
  static int configured_dev = -1;
  int dev = 0;
  KPX_CUDA_TRY(cudaGetDevice(&dev));
  auto kern = paged_decode_kernel<T, QH, HG>;
  if (configured_dev != dev) {
    KPX_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem));
    configured_dev = dev;
  }
  int grid = device_info().sm_count * C::kCtasPerSm;
  if (grid > kMaxGrid) grid = kMaxGrid;
  *grid_out = grid;
  kern<<<grid, C::kThreads, C::kSmem, stream>>>(p);
  KPX_CUDA_TRY(cudaGetLastError());
  decode_merge_kernel<T><<<p.batch * p.num_kv_heads, kD, 0, stream>>>(p, grid, C::kPartialFloats,
                                                                      HG * QH);
  return cuda_status(cudaGetLastError());
}

template <typename T>
int dispatch_decode(const DecodeParams& p, const DecodePlan& pl, cudaStream_t stream, int* grid) {
  if (pl.hg == 1) {
    if (pl.qh == 1) return launch_decode<T, 1, 1>(p, stream, grid);
    if (pl.qh == 2) return launch_decode<T, 2, 1>(p, stream, grid);
    return launch_decode<T, 4, 1>(p, stream, grid);
  }
  return launch_decode<T, 4, 2>(p, stream, grid);
}

}  // namespace
}  // namespace kpx

using namespace kpx;

extern "C" int64_t kpx_decode_workspace_bytes(int32_t batch, int32_t num_q_heads,
                                              int32_t num_kv_heads, int32_t head_size) {
  (void)batch;
  if (num_q_heads <= 0 || num_kv_heads <= 0 || head_size != kD || num_q_heads % num_kv_heads)
    return -1;
  // 2 partial slots per persistent CTA, each 8 heads x (128 + 2) floats at most
  return int64_t(kStatusBytes) + int64_t(2) * kMaxGrid * 8 * (kD + 2) * sizeof(float);
}

extern "C" int kpx_paged_decode(void* out, const void* q, const void* k_pool, const void* v_pool,
                                const kpx_kv_layout* layout, const int32_t* block_table,
                                int32_t max_blocks_per_seq, const int32_t* seq_lens,
                                int32_t len_bias, int32_t batch, int32_t num_q_heads, float scale,
                                void* workspace, int64_t workspace_bytes, void* stream) {
  if (!layout_ok(layout) || !out || !q || !k_pool || !v_pool || batch < 0 || num_q_heads <= 0)
    return KPX_ERR_INVALID_ARGUMENT;
  if (layout->head_size != kD || layout->block_size != kBS) return KPX_ERR_UNIMPLEMENTED;
  if (num_q_heads % layout->num_kv_heads) return KPX_ERR_INVALID_ARGUMENT;
  if (block_table && max_blocks_per_seq <= 0) return KPX_ERR_INVALID_ARGUMENT;
  if (!seq_lens && len_bias < 0) return KPX_ERR_INVALID_ARGUMENT;
  DecodePlan pl;
  if (!plan_for(num_q_heads / layout->num_kv_heads, &pl)) return KPX_ERR_UNIMPLEMENTED;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15)) return KPX_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool) |
       reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15)
    return KPX_ERR_INVALID_ARGUMENT;
  if (workspace_bytes <
      kpx_decode_workspace_bytes(batch, num_q_heads, layout->num_kv_heads, layout->head_size))
    return KPX_ERR_WORKSPACE_TOO_SMALL;
  if (batch == 0) return KPX_OK;
  if (!device_info().ok) return KPX_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int eb = elt_bytes(layout->dtype);
  DecodeParams p;
  p.k_pool = static_cast<const uint8_t*>(k_pool);
  p.v_pool = static_cast<const uint8_t*>(v_pool);
  p.status = static_cast<int32_t*>(workspace);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kStatusBytes);
  p.block_stride_b = layout->block_stride * eb;
  p.head_stride_b = layout->head_stride * eb;
  p.token_stride_b = layout->token_stride * eb;
  p.num_blocks = layout->num_blocks;
  p.max_blocks_per_seq = max_blocks_per_seq;
  p.len_bias = len_bias;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = layout->num_kv_heads;
  p.kv_mul = num_q_heads / layout->num_kv_heads;
  p.tile_contig = tile_contiguous(layout) ? 1 : 0;
  p.qscale = scale * kLog2e;
  // the prefix table of one launch lives in shared memory: long batches go in slices
  for (int32_t b0 = 0; b0 < batch; b0 += kMaxBatch) {
    int32_t nb = batch - b0 < kMaxBatch ? batch - b0 : kMaxBatch;
    p.batch = nb;
    p.out = static_cast<uint8_t*>(out) + int64_t(b0) * num_q_heads * kD * eb;
    p.q = static_cast<const uint8_t*>(q) + int64_t(b0) * num_q_heads * kD * eb;
    p.block_table = block_table ? block_table + int64_t(b0) * max_blocks_per_seq : nullptr;
    p.seq_lens = seq_lens ? seq_lens + b0 : nullptr;
    int grid = 0, rc;
    switch (layout->dtype) {
      case KPX_F16: rc = dispatch_decode<__half>(p, pl, s, &grid); break;
      case KPX_BF16: rc = dispatch_decode<__nv_bfloat16>(p, pl, s, &grid); break;
      default: rc = dispatch_decode<float>(p, pl, s, &grid); break;
    }
    if (rc != KPX_OK) return rc;
  }
  return KPX_OK;
}

