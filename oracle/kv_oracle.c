/*
 * kv_oracle.c -- CPU restatement of the kuiper fp32 attention / KV-cache path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against and the timed CPU baseline; nothing in the product library links,
 * loads or calls it.
 *
 * Parity status: pinned against the reference itself.  The reference ships no golden
 * vectors for attention, RoPE or the KV append (its tests for these pieces are commented
 * out and draw from an unseeded random_device), so the pin is the reference's own CPU
 * kernels run on seeded inputs: cpu/{mha,matmul,softmax,scale_sum,rope,rmsnorm}_kernel.cpp
 * with tensor.cpp and the allocator sources compile unmodified against small stand-ins
 * for their two third-party headers (oracle/shim/, oracle/ref_cpu_glue.cpp; Makefile target
 * `ref`), and tests/test_oracle_ref_cpu.py requires this file to reproduce their outputs
 * bit for bit when the stand-in's reductions run in index order, and within 1e-6 when
 * they run as Armadillo's own two-running-sums loops do.  The outputs are also committed
 * as tests/golden/ref_cpu_golden.npz for machines without the reference checkout.  The
 * integer paths (radix tree / prefix cache) are pinned separately against the reference
 * headers compiled directly.
 *
 * The Armadillo expressions at the reference call sites reduce to: a 128-long dot
 * product (fmat 1xK times Kx1), element-wise exp, a sum, a scalar*vector and a vector +=.
 * Armadillo does not define the summation order of the dot product (with a BLAS it is
 * the BLAS's), so orc_mha accumulates sequentially in fp32 and orc_mha_f64 gives a
 * float64 shadow to bound the oracle's own rounding error.
 *
 * Every function names the reference lines it follows (paths are relative to
 * the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* kuiper/source/op/kernels/cpu/rope_kernel.cpp:44-56 (Qwen branch; theta is a
 * runtime argument here, 1e6 for the Qwen2/Qwen3 builds, 5e5 for Llama3). */
ORC_API void orc_sin_cos_cache(int32_t head_size, int32_t max_seq_len, float theta,
                               float* sin_cache, float* cos_cache) {
  for (int32_t pos = 0; pos < max_seq_len; ++pos) {
    for (int32_t head_dim = 0; head_dim < head_size; ++head_dim) {
      float freq = 1.0f / powf(theta, (float)head_dim / (float)head_size);
      float val = (float)pos * freq;
      cos_cache[(int64_t)pos * head_size + head_dim] = cosf(val);
      sin_cache[(int64_t)pos * head_size + head_dim] = sinf(val);
    }
  }
}

/* kuiper/source/op/kernels/cpu/rope_kernel.cpp:58-82: half-split rotation of
 * the pairs (j, j + head_size/2) inside every head; sin/cos read at index
 * pos*head_size + 2*j; K is rotated only for head bases below kv_dim. */
ORC_API void orc_rope(int32_t dim, int32_t kv_dim, int32_t head_size, float* q, float* k,
                      int32_t pos, const float* sin_cache, const float* cos_cache) {
  for (int32_t i = 0; i < dim; i += head_size) {
    for (int32_t j = 0; j < head_size / 2; ++j) {
      float fci = sin_cache[(int64_t)pos * head_size + j * 2];
      float fcr = cos_cache[(int64_t)pos * head_size + j * 2];
      int32_t rotn = i < kv_dim ? 2 : 1;
      for (int32_t v = 0; v < rotn; ++v) {
        float* vec = v == 0 ? q : k;
        if (!vec) continue;
        float v0 = vec[i + j];
        float v1 = vec[i + j + head_size / 2];
        vec[i + j] = v0 * fcr - v1 * fci;
        vec[i + j + head_size / 2] = v0 * fci + v1 * fcr;
      }
    }
  }
}

/* RoPE over a chunk of n tokens at positions start_pos .. start_pos+n-1, the
 * CPU statement of what kuiper/source/op/kernels/cuda/rope_kernel.cu:327-375
 * (batched_rope_kernel_cu_fp32) computes: orc_rope per row. */
ORC_API void orc_rope_batched(int32_t start_pos, int32_t n, int32_t dim, int32_t kv_dim,
                              int32_t head_size, float* q, float* k, const float* sin_cache,
                              const float* cos_cache) {
  for (int32_t s = 0; s < n; ++s) {
    orc_rope(dim, kv_dim, head_size, q ? q + (int64_t)s * dim : NULL,
             k ? k + (int64_t)s * kv_dim : NULL, start_pos + s, sin_cache, cos_cache);
  }
}

/* Per-head RMSNorm of n rows of `heads` heads (Qwen3 q/k norm before RoPE), in place:
 * kuiper/source/op/kernels/cpu/rmsnorm_kernel.cpp:26-34 applied to every head row
 * (kuiper/source/model/qwen3.cpp:1019-1034 reshapes q / k to [heads, head_size] and
 * calls it): mean = mean(x^2) + eps; out = w * ((1/sqrt(mean)) * x).  The mean is
 * accumulated sequentially in fp32 (Armadillo's order is unspecified). */
ORC_API void orc_rmsnorm_heads(float* x, int64_t rows, int32_t heads, int32_t head_size,
                               const float* weight, float eps) {
  for (int64_t r = 0; r < rows * heads; ++r) {
    float* row = x + r * head_size;
    float sum = 0.f;
    for (int32_t i = 0; i < head_size; ++i) sum += row[i] * row[i];
    const float mean = sum / (float)head_size + eps;
    const float rs = 1.f / sqrtf(mean);
    for (int32_t i = 0; i < head_size; ++i) row[i] = weight[i] * (rs * row[i]);
  }
}

/* kuiper/source/op/kernels/cpu/softmax_kernel.cpp:4-15 */
static void softmax_inplace(float* x, int32_t size) {
  float max_value = x[0];
  for (int32_t i = 1; i < size; ++i)
    if (x[i] > max_value) max_value = x[i];
  float sum_value = 0.f;
  for (int32_t i = 0; i < size; ++i) {
    x[i] = expf(x[i] - max_value);
    sum_value += x[i];
  }
  for (int32_t i = 0; i < size; ++i) x[i] = x[i] / sum_value;
}

ORC_API void orc_softmax_inplace(float* x, int32_t size) { softmax_inplace(x, size); }

/* One head of kuiper/source/op/kernels/cpu/mha_kernel.cpp:19-60.
 *  :28-39  score[t] = (q . k_t) * scale        (cpu/matmul_kernel.cpp:37-40)
 *  :41-44  softmax over pos+1 scores           (cpu/softmax_kernel.cpp:4-15)
 *  :46-59  out = 0; out += score[t] * v_t, t ascending (cpu/scale_sum_kernel.cpp:17-21) */
static void mha_one_head(int32_t h, int32_t pos, int32_t seq_len, int32_t kv_dim, int32_t kv_mul,
                         int32_t head_size, int64_t layer_offset, float scale, float* out,
                         const float* q, float* score, const float* kc, const float* vc) {
  float* score_head = score + (int64_t)h * seq_len;
  const float* qh = q + (int64_t)h * head_size;
  for (int32_t t = 0; t <= pos; ++t) {
    int64_t cache_offset = (int64_t)t * kv_dim + (int64_t)(h / kv_mul) * head_size;
    const float* kh = kc + layer_offset + cache_offset;
    float dot = 0.f;
    for (int32_t i = 0; i < head_size; ++i) dot += qh[i] * kh[i];
    score_head[t] = dot * scale;
  }
  softmax_inplace(score_head, pos + 1);
  float* oh = out + (int64_t)h * head_size;
  memset(oh, 0, sizeof(float) * head_size);
  const float* vh = vc + layer_offset + (int64_t)(h / kv_mul) * head_size;
  for (int32_t t = 0; t <= pos; ++t) {
    float s = score_head[t];
    const float* vt = vh + (int64_t)t * kv_dim;
    for (int32_t i = 0; i < head_size; ++i) oh[i] += s * vt[i];
  }
}

/* kuiper/source/op/kernels/cpu/mha_kernel.cpp:5-61 with the same argument list
 * as kernel::MHAKernel (kernels_interface.h:22-28), raw pointers in place of
 * Tensors.  The reference computes layer_offset in int32 (:10); it is int64
 * here so pool-sized caches do not overflow (same value wherever the reference
 * does not overflow).  Single thread, head loop outermost as in the reference. */
ORC_API void orc_mha(int32_t pos, int32_t head_num, int32_t layer_index, int32_t seq_len,
                     int32_t kv_dim, int32_t kv_mul, int32_t head_size, float* mha_out,
                     const float* query, float* score, const float* key_cache,
                     const float* value_cache) {
  int64_t layer_offset = (int64_t)layer_index * seq_len * kv_dim;
  float scale = 1.f / sqrtf((float)head_size);
  for (int32_t h = 0; h < head_num; ++h)
    mha_one_head(h, pos, seq_len, kv_dim, kv_mul, head_size, layer_offset, scale, mha_out, query,
                 score, key_cache, value_cache);
}

/* float64 shadow of orc_mha: same formula, all arithmetic in double.  Used to
 * report how far the fp32 oracle itself is from the exact result. */
ORC_API void orc_mha_f64(int32_t pos, int32_t head_num, int32_t layer_index, int32_t seq_len,
                         int32_t kv_dim, int32_t kv_mul, int32_t head_size, double* mha_out,
                         const float* query, const float* key_cache, const float* value_cache) {
  int64_t layer_offset = (int64_t)layer_index * seq_len * kv_dim;
  double scale = 1.0 / sqrt((double)head_size);
  double* sc = (double*)malloc(sizeof(double) * (size_t)(pos + 1));
  for (int32_t h = 0; h < head_num; ++h) {
    const float* qh = query + (int64_t)h * head_size;
    double mx = -INFINITY;
    for (int32_t t = 0; t <= pos; ++t) {
      const float* kh = key_cache + layer_offset + (int64_t)t * kv_dim + (int64_t)(h / kv_mul) * head_size;
      double dot = 0.0;
      for (int32_t i = 0; i < head_size; ++i) dot += (double)qh[i] * (double)kh[i];
      sc[t] = dot * scale;
      if (sc[t] > mx) mx = sc[t];
    }
    double sum = 0.0;
    for (int32_t t = 0; t <= pos; ++t) {
      sc[t] = exp(sc[t] - mx);
      sum += sc[t];
    }
    double* oh = mha_out + (int64_t)h * head_size;
    for (int32_t i = 0; i < head_size; ++i) oh[i] = 0.0;
    for (int32_t t = 0; t <= pos; ++t) {
      double s = sc[t] / sum;
      const float* vt = value_cache + layer_offset + (int64_t)t * kv_dim + (int64_t)(h / kv_mul) * head_size;
      for (int32_t i = 0; i < head_size; ++i) oh[i] += s * (double)vt[i];
    }
  }
  free(sc);
}

/* Causal attention of n queries at positions start_pos..start_pos+n-1 against
 * cache rows 0..start_pos+i: the CPU statement of batched_mha_kernel_cu
 * (kuiper/source/op/kernels/cuda/mha_kernel.cu:347-444; cur_pos = start_pos +
 * seq_idx) -- orc_mha once per query row.  query/out are [n, head_num*head_size];
 * score is scratch of head_num*seq_len floats per thread.  threads > 1 spreads
 * the query rows over OpenMP threads (results do not depend on it). */
ORC_API void orc_mha_prefill(int32_t start_pos, int32_t n, int32_t head_num, int32_t layer_index,
                             int32_t seq_len, int32_t kv_dim, int32_t kv_mul, int32_t head_size,
                             float* out, const float* query, const float* key_cache,
                             const float* value_cache, int32_t threads) {
  int64_t dim = (int64_t)head_num * head_size;
  (void)threads;
#ifdef _OPENMP
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
#endif
  {
    float* score = (float*)malloc(sizeof(float) * (size_t)head_num * (size_t)seq_len);
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 4)
#endif
    for (int32_t s = 0; s < n; ++s) {
      orc_mha(start_pos + s, head_num, layer_index, seq_len, kv_dim, kv_mul, head_size,
              out + s * dim, query + s * dim, score, key_cache, value_cache);
    }
    free(score);
  }
}

/* The reference append is a row copy: cache[layer][pos][:] = src
 * (kuiper/source/op/kernels/cuda/kv_cache_kernel.cu:13-25; the eager path writes
 * the projection straight into the row, kuiper/source/model/model.cpp:348-385). */
ORC_API void orc_append_contiguous(float* cache, const float* src, int32_t pos, int32_t kv_dim,
                                   int32_t layer_idx, int32_t seq_len) {
  memcpy(cache + (int64_t)layer_idx * seq_len * kv_dim + (int64_t)pos * kv_dim, src,
         sizeof(float) * (size_t)kv_dim);
}

/* ---- paged view (no reference counterpart; this is the spec the CUDA path is
 * held to).  A pool is [num_blocks][kv_heads][block_size][head_size]; the slot of
 * (block, offset) is block*block_size + offset.  elt_bytes-wide elements are
 * moved as raw bytes so fp16 / bf16 / fp32 pools are all bit-exact copies. ---- */

ORC_API void orc_append_paged(uint8_t* pool, const uint8_t* src, const int64_t* slot_mapping,
                              int32_t num_tokens, int32_t kv_heads, int32_t head_size,
                              int32_t block_size, int32_t elt_bytes) {
  size_t row = (size_t)head_size * (size_t)elt_bytes;
  for (int32_t t = 0; t < num_tokens; ++t) {
    int64_t slot = slot_mapping[t];
    if (slot < 0) continue; /* padding token: skipped */
    int64_t blk = slot / block_size, off = slot % block_size;
    for (int32_t h = 0; h < kv_heads; ++h) {
      uint8_t* dst = pool + (((blk * kv_heads + h) * block_size + off) * (int64_t)row);
      memcpy(dst, src + ((int64_t)t * kv_heads + h) * (int64_t)row, row);
    }
  }
}

/* Gather one sequence's first `len` tokens through its block-table row into the
 * reference's contiguous token-major layout [len, kv_heads*head_size], so that
 * orc_mha can be run on paged state unchanged. */
ORC_API void orc_gather_paged(uint8_t* dst, const uint8_t* pool, const int32_t* block_table_row,
                              int32_t len, int32_t kv_heads, int32_t head_size,
                              int32_t block_size, int32_t elt_bytes) {
  size_t row = (size_t)head_size * (size_t)elt_bytes;
  for (int32_t t = 0; t < len; ++t) {
    int64_t blk = block_table_row[t / block_size], off = t % block_size;
    for (int32_t h = 0; h < kv_heads; ++h) {
      const uint8_t* s = pool + (((blk * kv_heads + h) * block_size + off) * (int64_t)row);
      memcpy(dst + ((int64_t)t * kv_heads + h) * (int64_t)row, s, row);
    }
  }
}

/* Batched decode over paged fp32 pools: for each sequence gather to contiguous
 * and run orc_mha with pos = seq_len-1.  out/q are [batch, head_num*head_size].
 * threads > 1 spreads sequences over OpenMP threads. */
ORC_API void orc_paged_decode(float* out, const float* q, const float* k_pool, const float* v_pool,
                              const int32_t* block_table, int32_t max_blocks_per_seq,
                              const int32_t* seq_lens, int32_t batch, int32_t head_num,
                              int32_t kv_heads, int32_t head_size, int32_t block_size,
                              int32_t threads) {
  int32_t kv_dim = kv_heads * head_size, kv_mul = head_num / kv_heads;
  int64_t dim = (int64_t)head_num * head_size;
  (void)threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
#endif
  for (int32_t b = 0; b < batch; ++b) {
    int32_t len = seq_lens[b];
    if (len <= 0) {
      memset(out + b * dim, 0, sizeof(float) * (size_t)dim);
      continue;
    }
    float* kc = (float*)malloc(sizeof(float) * (size_t)len * kv_dim);
    float* vc = (float*)malloc(sizeof(float) * (size_t)len * kv_dim);
    float* score = (float*)malloc(sizeof(float) * (size_t)head_num * (size_t)len);
    const int32_t* row = block_table + (int64_t)b * max_blocks_per_seq;
    orc_gather_paged((uint8_t*)kc, (const uint8_t*)k_pool, row, len, kv_heads, head_size, block_size, 4);
    orc_gather_paged((uint8_t*)vc, (const uint8_t*)v_pool, row, len, kv_heads, head_size, block_size, 4);
    orc_mha(len - 1, head_num, 0, len, kv_dim, kv_mul, head_size, out + b * dim, q + b * dim,
            score, kc, vc);
    free(kc);
    free(vc);
    free(score);
  }
}

ORC_API int32_t orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
