/*
 * kpx.h -- C ABI of the B200 (sm_100a) KV-cache path for the kuiper operator API.
 *
 * Every entry point takes plain device/host pointers, integer sizes and a CUDA
 * stream passed as void* (cudaStream_t); none allocates unless it says so, none
 * synchronises the stream unless it says so, none aborts: the return value is a
 * status code (0 = KPX_OK).  There is no CPU fallback: on a machine without a
 * CUDA device the compute entry points return KPX_ERR_CUDA.
 *
 * Each declaration cites the interface of the reference project (paths relative
 * to its root) that it stands in for.
 */
#ifndef KPX_H_
#define KPX_H_
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KPX_API __attribute__((visibility("default")))

/* Status codes.  0,1,5,7 keep the numeric values of base::StatusCode
 * (kuiper/include/base/base.h:96-104) so the C++ adapters can forward them. */
enum {
  KPX_OK = 0,
  KPX_ERR_UNIMPLEMENTED = 1,
  KPX_ERR_INTERNAL = 5,
  KPX_ERR_INVALID_ARGUMENT = 7,
  KPX_ERR_OUT_OF_BLOCKS = 8,
  KPX_ERR_CUDA = 9,
  KPX_ERR_WORKSPACE_TOO_SMALL = 10,
  KPX_ERR_DEVICE_TIMEOUT = 11,
  KPX_ERR_REFCOUNT = 12,
  KPX_ERR_NOT_FOUND = 13,
  KPX_ERR_STATIC_SCRATCH_LIMIT = 14
};

/* Element types of pools, queries and outputs (base::DataType has Fp32 and Fp16,
 * kuiper/include/base/base.h:58-64; bf16 is an addition). */
enum { KPX_F16 = 0, KPX_BF16 = 1, KPX_F32 = 2 };

/* Addressing of a K or V cache for one layer.  Element (block, head, token, i)
 * lives at  base + block*block_stride + head*head_stride + token*token_stride + i
 * (strides in elements, int64 throughout).
 *   paged pool  [num_blocks][kv_heads][block_size][head_size]:
 *       block_stride = kv_heads*block_size*head_size, head_stride = block_size*head_size,
 *       token_stride = head_size          -> one (block, head) tile is contiguous
 *   reference cache [seq_len][kv_heads*head_size] (kuiper/source/model/model.cpp:348-385),
 *   seen as blocks of block_size consecutive rows with an identity block table:
 *       block_stride = block_size*kv_dim, head_stride = head_size, token_stride = kv_dim */
typedef struct kpx_kv_layout {
  int32_t dtype;        /* KPX_F16 | KPX_BF16 | KPX_F32 */
  int32_t num_kv_heads;
  int32_t head_size;    /* 128 */
  int32_t block_size;   /* 16 tokens */
  int64_t block_stride;
  int64_t head_stride;
  int64_t token_stride;
  int64_t num_blocks;   /* blocks addressable from base; 0 = unknown (ids are not range-checked) */
} kpx_kv_layout;

KPX_API const char* kpx_status_string(int status);
KPX_API int kpx_abi_version(void);
KPX_API int kpx_device_count(void);

/* Fill *out with the paged-pool layout / with the reference's contiguous layout. */
KPX_API int kpx_layout_paged(kpx_kv_layout* out, int32_t dtype, int32_t num_kv_heads,
                             int32_t head_size, int32_t block_size);
KPX_API int kpx_layout_contiguous(kpx_kv_layout* out, int32_t dtype, int32_t num_kv_heads,
                                  int32_t head_size, int32_t block_size);

/* ---------------------------------------------------------------- append ----
 * Scatter num_tokens rows of K and V ([num_tokens, kv_heads*head_size], already
 * RoPE'd) into the cache: token t goes to slot slot_mapping[t] (= block*block_size
 * + offset; negative = skip).  If slot_mapping is NULL the rows go to consecutive
 * slots starting at *pos_dev (a device int32, the reference's GPU-resident
 * position) plus pos_bias.  Bit-exact copy, 128-bit vectorised.
 * Replaces copy_to_kv_cache_kernel / _fp16 (kuiper/source/op/kernels/cuda/
 * kv_cache_kernel.cuh:24-33), fused_kv_cache_update_cu (cuda/fused_kernels.cuh:53-64)
 * and the prefill cudaMemcpyAsync pair (kuiper/source/model/qwen3.cpp:1224-1241).
 * v_pool/v_src may be NULL to append K only (KVCacheLayer appends one at a time). */
KPX_API int kpx_append(void* k_pool, void* v_pool, const kpx_kv_layout* layout, const void* k_src,
                       const void* v_src, const int64_t* slot_mapping, const int32_t* pos_dev,
                       int32_t pos_bias, int32_t num_tokens, void* stream);

/* RoPE (half-split pairs (j, j+head_size/2), fp32 math, one rounding at the store)
 * on num_tokens rows of Q [num_tokens, q_heads*head_size] and K, in place, with
 * sin/cos read from fp32 tables [max_pos, head_size] at index pos*head_size + 2j;
 * then, if k_pool is not NULL, the rotated K rows and the V rows are appended as
 * kpx_append does.  Token t sits at position positions[t] + pos_base (positions: device
 * int32 [num_tokens]) or, with positions NULL, at pos_base + t (a chunk starting at
 * pos_base, the reference's batched RoPE).  The products
 * are not contracted into FMAs, so the result is bit-identical to the reference
 * CPU statement when both read the same tables.
 * Replaces rope_kernel_cu / _gpu_pos / _fp16_gpu_pos / batched_rope_kernel_cu
 * (kuiper/source/op/kernels/cuda/rope_kernel.cuh:5-28), CPU statement
 * kuiper/source/op/kernels/cpu/rope_kernel.cpp:58-82.  q or k may be NULL. */
KPX_API int kpx_rope_append(void* q, void* k, const void* v, int32_t q_heads,
                            const int32_t* positions, int32_t pos_base, const float* sin_cache,
                            const float* cos_cache, void* k_pool, void* v_pool,
                            const kpx_kv_layout* layout, const int64_t* slot_mapping,
                            int32_t num_tokens, void* stream);

/* kpx_rope_append with the per-head RMSNorm of Qwen3 in front of the rotation: every head row
 * x of Q (weights q_norm_weight) and of K (k_norm_weight), both fp32 [head_size], becomes
 * w * (x / sqrt(mean(x^2) + norm_eps)) in fp32 before it is rotated; the row is rounded to the
 * cache dtype once, after the rotation.  A NULL weight pointer leaves that tensor unnormalised;
 * with both NULL this is kpx_rope_append.
 * Replaces the sequence RmsNorm(q) -> RmsNorm(k) -> RoPE -> cache store of the Qwen3 attention
 * block (kuiper/source/model/qwen3.cpp:1019-1046,1090-1126; rmsnorm statement
 * kuiper/source/op/kernels/cpu/rmsnorm_kernel.cpp:26-34, eps 1e-6 for Qwen). */
KPX_API int kpx_norm_rope_append(void* q, void* k, const void* v, int32_t q_heads,
                                 const float* q_norm_weight, const float* k_norm_weight, float norm_eps,
                                 const int32_t* positions, int32_t pos_base, const float* sin_cache,
                                 const float* cos_cache, void* k_pool, void* v_pool,
                                 const kpx_kv_layout* layout, const int64_t* slot_mapping,
                                 int32_t num_tokens, void* stream);

/* fp32 sin/cos tables [max_seq_len, head_size]: table[pos*head_size + k] =
 * sin/cos(pos * theta^(-k/head_size)).  Replaces sin_cos_cache_calc_cu
 * (kuiper/source/op/kernels/cuda/rope_kernel.cuh:22-23). */
KPX_API int kpx_sin_cos_cache(float* sin_cache, float* cos_cache, int32_t head_size,
                              int32_t max_seq_len, float theta, void* stream);

/* ---------------------------------------------------------------- decode ----
 * Bytes of device scratch kpx_paged_decode needs on the current device for up
 * to `batch` sequences (split-KV partials of the persistent CTAs + a status
 * word).  Does not depend on sequence lengths. */
KPX_API int64_t kpx_decode_workspace_bytes(int32_t batch, int32_t num_q_heads,
                                           int32_t num_kv_heads, int32_t head_size);

/* Single-query attention for `batch` sequences: out[b,h,:] = softmax(scale *
 * q[b,h,:] . K[b, 0..len_b-1, h/kv_mul, :]) V[...], K/V gathered through
 * block_table[b][0..] (int32 [batch, max_blocks_per_seq] on the device; NULL =
 * identity table 0,1,2,... which is the reference's contiguous cache).
 * len_b = seq_lens[b] + len_bias with seq_lens a device int32 array (the
 * reference's device-resident pos: pass len_bias = 1); if seq_lens is NULL every
 * sequence has len_bias tokens.  q/out are [batch, num_q_heads*head_size] of the
 * layout's dtype.  len_b = 0 gives zeros.  All variable state is read from device
 * memory and the shared-memory size is fixed, so the launch can be captured.
 * Replaces mha_kernel_cu / _gpu_pos (kuiper/source/op/kernels/cuda/mha_kernel.cuh:4-18),
 * flash_attention_decode[_fp16][_gpu_pos]_cu and flash_attention2_decode* (cuda/
 * flash_attention_kernel.cuh:47-61,92-126,181-234); arithmetic statement: cpu/
 * mha_kernel.cpp:5-61. */
KPX_API int kpx_paged_decode(void* out, const void* q, const void* k_pool, const void* v_pool,
                             const kpx_kv_layout* layout, const int32_t* block_table,
                             int32_t max_blocks_per_seq, const int32_t* seq_lens,
                             int32_t len_bias, int32_t batch, int32_t num_q_heads, float scale,
                             void* workspace, int64_t workspace_bytes, void* stream);

/* kpx_paged_decode for launches that the caller overlaps on the GPU with other launches of
 * this library (consecutive layers or requests on different streams, each launch with ITS OWN
 * workspace).  Same arguments and results.  The kernel then runs as three CTAs of four warps per
 * SM instead of one CTA of twelve, so that an SM passes from one launch to the next a third at
 * a time while the earlier launch's last warps finish; run alone, kpx_paged_decode's single
 * large CTA is the faster form.  No reference counterpart (the reference runs one kernel at a
 * time on one stream). */
KPX_API int kpx_paged_decode_overlapped(void* out, const void* q, const void* k_pool, const void* v_pool,
                                        const kpx_kv_layout* layout, const int32_t* block_table,
                                        int32_t max_blocks_per_seq, const int32_t* seq_lens,
                                        int32_t len_bias, int32_t batch, int32_t num_q_heads, float scale,
                                        void* workspace, int64_t workspace_bytes, void* stream);

/* Plan of a decode step.  All launches of one step (one per layer) see the same lengths and the
 * same block table, so what each of them works out in its prologue (the block prefix over the
 * sequences, every warp's starting point on the line of blocks, the id of its first block) is
 * the same for all of them.  kpx_decode_plan works it out once into `plan` (device memory, 16-byte
 * aligned, kpx_decode_plan_bytes() bytes); kpx_paged_decode_planned is kpx_paged_decode (flags 0)
 * or kpx_paged_decode_overlapped (flags KPX_DECODE_OVERLAPPED) with that plan: a CTA then starts
 * streaming after one load instead of three dependent ones.  Results are bit-identical with and
 * without a plan.  The plan must have been made, earlier on the same stream or otherwise ordered
 * before the launch, from the SAME block_table, seq_lens contents, len_bias, batch, head counts
 * and cache dtype: make it again whenever a length or a table entry changes (every step).  A
 * plan the launch cannot use (another batch or head layout, a batch of more than 512 sequences,
 * a launch small enough for the short-range form, plan == NULL) is ignored and the launch works
 * everything out itself; a plan that is out of date in its CONTENTS is the caller's error and is
 * not detected.  A length in the plan that the table rows cannot hold raises the status word of
 * the launch.  Capturable like kpx_paged_decode.  No reference counterpart (the reference
 * passes one position per launch). */
KPX_API int64_t kpx_decode_plan_bytes(void);
KPX_API int kpx_decode_plan(void* plan, int64_t plan_bytes, const kpx_kv_layout* layout,
                            const int32_t* block_table, int32_t max_blocks_per_seq, const int32_t* seq_lens,
                            int32_t len_bias, int32_t batch, int32_t num_q_heads, void* stream);
KPX_API int kpx_paged_decode_planned(void* out, const void* q, const void* k_pool, const void* v_pool,
                                     const kpx_kv_layout* layout, const int32_t* block_table,
                                     int32_t max_blocks_per_seq, const int32_t* seq_lens, int32_t len_bias,
                                     int32_t batch, int32_t num_q_heads, float scale, void* workspace,
                                     int64_t workspace_bytes, const void* plan, int32_t flags, void* stream);

/* One whole decode step of a layer in one launch: RoPE of the new token's Q and K rows,
 * append of its K / V rows to the pool, and the attention of kpx_paged_decode over the cached
 * tokens plus the new one.  positions[b] (device int32) is both the number of tokens sequence
 * b already has in the pool and the position of its new token; q [batch, num_q_heads*head_size],
 * k_new / v_new [batch, kv_heads*head_size] are read (not rotated in place); sin/cos tables as in
 * kpx_rope_append.  The new token goes to row positions[b] % block_size of block
 * block_table[b][positions[b] / block_size] (identity table if NULL), stored with the same bits
 * kpx_rope_append stores; the attention takes it from registers, so the launch never reads what
 * it writes.  Each (sequence, kv head) row pair is stored by the warp that finishes that
 * sequence's last cached block.  Workspace, status word and capture rules as kpx_paged_decode.
 * flags: KPX_DECODE_OVERLAPPED when the caller runs this launch concurrently with other launches
 * of this library (another stream, ANOTHER workspace): the kernel then uses three small CTAs per
 * SM so that SMs pass from one launch to the next in thirds; 0 otherwise.
 * Replaces the decode-step sequence RoPEGpuPosLayer -> KVCacheLayer(K), KVCacheLayer(V) ->
 * FlashAttentionDecodeLayer / MHAGpuPosLayer of attention_qkv_with_graph and
 * attention_mha_with_graph (kuiper/source/model/qwen3.cpp:1052-1127,
 * kuiper/source/model/qwen_base.cpp:145-192). */
enum { KPX_DECODE_OVERLAPPED = 1 };
KPX_API int kpx_rope_append_decode(void* out, const void* q, const void* k_new, const void* v_new,
                                   const float* sin_cache, const float* cos_cache, void* k_pool,
                                   void* v_pool, const kpx_kv_layout* layout,
                                   const int32_t* block_table, int32_t max_blocks_per_seq,
                                   const int32_t* positions, int32_t batch, int32_t num_q_heads,
                                   float scale, void* workspace, int64_t workspace_bytes,
                                   int32_t flags, void* stream);

/* kpx_paged_decode for callers that cannot allocate or pass scratch memory: a plugin
 * inside a host that owns the device heap, a kernel registry whose signature carries only
 * inputs and outputs (the reference's MHAKernel is one), code that may not call cudaMalloc
 * between steps.  Same arguments and results as kpx_paged_decode minus the workspace; the
 * scratch is a 10 715 392-byte array built into the library, which every GPU that loads
 * the library holds until the process exits.  It allocates nothing (no cudaMalloc /
 * cudaFree / allocating library call).
 * Limits: num_kv_heads * ceil(kv_mul / 4) <= 16 (kv_mul = num_q_heads / num_kv_heads; for
 * kv_mul 1 or 2 the factor is 1); anything larger returns KPX_ERR_STATIC_SCRATCH_LIMIT.
 * The first call on each device looks up the array's device address (and sets kernel
 * attributes); make that first call before any stream capture.  All calls on a device
 * share the one array: calls that overlap on the GPU (different streams) race and must be
 * serialised by the caller; calls on one stream are fine.  The status word is cleared at
 * the start of every call and is not readable through this entry point.
 * This entry point has no counterpart in the reference. */
KPX_API int kpx_paged_decode_static(void* out, const void* q, const void* k_pool,
                                    const void* v_pool, const kpx_kv_layout* layout,
                                    const int32_t* block_table, int32_t max_blocks_per_seq,
                                    const int32_t* seq_lens, int32_t len_bias, int32_t batch,
                                    int32_t num_q_heads, float scale, void* stream);

/* A workspace starts with a 256-byte header whose first word is a sticky status
 * the kernels raise (never clear).  kpx_workspace_init zeroes the header (async on
 * `stream`); call it once after allocating a workspace.  kpx_workspace_status
 * synchronises the stream, returns the word -- KPX_OK, KPX_ERR_DEVICE_TIMEOUT if a
 * bounded device-side wait gave up, KPX_ERR_INVALID_ARGUMENT if a block id outside
 * [0, layout.num_blocks) was met -- and clears it.  After KPX_ERR_DEVICE_TIMEOUT the launch
 * that raised it has left rows of its output unwritten and piece counters in the workspace
 * half counted, so the workspace has to start over before its next launch.
 * kpx_workspace_status does that itself when it reads this code (it wipes the workspace to the
 * size kpx_workspace_init was given); a caller that watches the word by other means calls
 * kpx_workspace_init again.  Then repeat the step.  No reference counterpart (the reference does not check its launches on the hot
 * path; its only recovery is the eager fallback after a failed graph capture,
 * kuiper/source/model/qwen_base.cpp:754). */
KPX_API int kpx_workspace_init(void* workspace, int64_t workspace_bytes, void* stream);
KPX_API int kpx_workspace_status(void* workspace, void* stream);

/* --------------------------------------------------------------- prefill ----
 * Causal attention of a chunk of queries against the cache the chunk has
 * already been appended to.  Sequence b owns query rows
 * [cu_q_lens[b], cu_q_lens[b+1]) of q/out ([total_q, num_q_heads*head_size]);
 * its query i sits at position start_pos[b] + i and attends cache positions
 * 0 .. start_pos[b]+i.  cu_q_lens (int32 [batch+1]) and start_pos (int32 [batch])
 * are HOST arrays (they size the grid).
 * Replaces batched_mha_kernel_cu (kuiper/source/op/kernels/cuda/mha_kernel.cuh:20-26),
 * flash_attention_prefill[_fp16]_cu, flash_attention2_prefill[_fp16]_cu (cuda/
 * flash_attention_kernel.cuh:27-42,71-86,139-174). */
KPX_API int64_t kpx_prefill_workspace_bytes(int32_t total_q, int32_t num_q_heads,
                                            int32_t num_kv_heads, int32_t head_size);
KPX_API int kpx_paged_prefill(void* out, const void* q, const void* k_pool, const void* v_pool,
                              const kpx_kv_layout* layout, const int32_t* block_table,
                              int32_t max_blocks_per_seq, const int32_t* cu_q_lens_host,
                              const int32_t* start_pos_host, int32_t batch, int32_t num_q_heads,
                              float scale, void* workspace, int64_t workspace_bytes, void* stream);

/* ------------------------------------------------- block sharing on device --
 * Copy-on-write: for i < n copy block src_ids[i] to block dst_ids[i] in the K and
 * the V pool of every layer (pools of consecutive layers are layer_stride
 * elements apart).  src_ids/dst_ids are device int32 arrays.  No reference
 * counterpart (the reference cache is never shared between sequences). */
KPX_API int kpx_cow_copy_blocks(void* k_pool, void* v_pool, const kpx_kv_layout* layout,
                                int32_t num_layers, int64_t layer_stride, const int32_t* src_ids,
                                const int32_t* dst_ids, int32_t n, void* stream);

/* refcounts[block_ids[i]] += deltas[i] for i < n (device arrays; duplicates
 * allowed).  A count that would go below zero, or a block id outside
 * [0, num_blocks), is left untouched and recorded: *error_count_dev (device
 * int32, may be NULL) is incremented.  No reference counterpart (the reference
 * counts references per radix node on the host, radix_tree.h:158-178). */
KPX_API int kpx_refcount_update(int32_t* refcounts, int32_t num_blocks, const int32_t* block_ids,
                                const int32_t* deltas, int32_t n, int32_t* error_count_dev,
                                void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KPX_H_ */
