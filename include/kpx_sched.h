/*
 * kpx_sched.h -- C ABI of the request scheduler over the paged KV cache
 * (lib/libkuiper_b200.so; C++ class base::KVScheduler in kuiper/base/kv_scheduler.h).
 *
 * Reference interfaces this stands in for: the per-request flow of generate_response
 * (demo/inference_common.h:1050-1262: match -> incremental prefill from the matched position
 * -> decode loop -> register_prefix -> release) and PrefixCacheManager (:757-853).  The
 * reference serves one request at a time; batching many requests, chunking their prefill and
 * gating admission by free blocks have no reference counterpart.
 *
 * A step is fetched as plain host arrays, sized by kpx_sched_*_shape first, and handed to
 * kpx_rope_append / kpx_append, kpx_paged_prefill and kpx_paged_decode of kpx.h.
 */
#ifndef KPX_SCHED_H_
#define KPX_SCHED_H_
#include <stdint.h>

#include "kpx_kvm.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kpx_sched kpx_sched;

/* The scheduler works on the pool and prefix cache of `kvm` (not owned; must outlive it). */
KPX_API kpx_sched* kpx_sched_create(kpx_kvm* kvm, int32_t prefill_chunk, int32_t max_prefill_tokens,
                                    int32_t max_prefill_rows, int32_t max_decode_batch,
                                    int32_t use_prefix_cache);
KPX_API void kpx_sched_destroy(kpx_sched* s);

/* -> request id >= 0, or -1 on bad arguments.  also_register > 0: at the end the first
 * also_register tokens are registered as a prefix of their own too (a shared system prompt). */
KPX_API int32_t kpx_sched_submit(kpx_sched* s, const int32_t* prompt, int32_t prompt_len, int32_t max_new_tokens,
                                 int32_t also_register);
/* One turn of a conversation (the reference's end-of-turn fix-up, demo/inference_common.h:
 * 1334-1358): when generation ends, the last sampled token and the suffix_len >= 0 tokens the
 * chat template puts after it are prefilled as well (rows with completes == 0, nothing is
 * sampled), and the whole history is registered, so that the next turn's prompt hits all of it.
 * The request is in state 4 (gap fill) meanwhile. */
KPX_API int32_t kpx_sched_submit_turn(kpx_sched* s, const int32_t* prompt, int32_t prompt_len,
                                      int32_t max_new_tokens, int32_t also_register,
                                      const int32_t* turn_suffix, int32_t suffix_len);
/* Sampled tokens that end a request before max_new_tokens (the reference's
 * model.is_sentence_ending, demo/inference_common.h:1204); n = 0 clears the set.  The end
 * token is kept as the request's last token (it has no K/V unless the turn's gap is filled). */
KPX_API int kpx_sched_set_end_tokens(kpx_sched* s, const int32_t* token_ids, int32_t n);
/* -> number of requests moved from waiting to running. */
KPX_API int32_t kpx_sched_admit(kpx_sched* s);

/* Prefill: build the next step (-> 1, or 0 when nothing is left to prefill), read its shape,
 * copy its arrays out (any pointer may be NULL), report the sampled tokens (one per row; only
 * rows with completes[row] == 1 are read). */
KPX_API int kpx_sched_next_prefill(kpx_sched* s);
KPX_API int kpx_sched_prefill_shape(const kpx_sched* s, int32_t* rows, int32_t* tokens, int32_t* max_blocks);
KPX_API int kpx_sched_prefill_arrays(const kpx_sched* s, int32_t* request_ids, int32_t* cu_q_lens,
                                     int32_t* start_pos, int32_t* positions, int64_t* slot_mapping,
                                     int32_t* token_ids, int32_t* completes, int32_t* block_table,
                                     int32_t max_blocks);
KPX_API int kpx_sched_complete_prefill(kpx_sched* s, const int32_t* sampled, int32_t rows);

/* Decode: the same round trip. */
KPX_API int kpx_sched_next_decode(kpx_sched* s);
KPX_API int kpx_sched_decode_shape(const kpx_sched* s, int32_t* rows, int32_t* max_blocks);
KPX_API int kpx_sched_decode_arrays(const kpx_sched* s, int32_t* request_ids, int32_t* seq_lens,
                                    int32_t* positions, int64_t* slot_mapping, int32_t* token_ids,
                                    int32_t* block_table, int32_t max_blocks);
KPX_API int kpx_sched_complete_decode(kpx_sched* s, const int32_t* sampled, int32_t rows);

/* Requests.  state: 0 waiting, 1 prefill, 2 decode, 3 finished (also: unknown id), 4 gap fill. */
KPX_API int32_t kpx_sched_state(const kpx_sched* s, int32_t request);
KPX_API int32_t kpx_sched_reused_tokens(const kpx_sched* s, int32_t request);
/* prompt followed by the generated tokens (then the turn's suffix, once the turn has ended);
 * -> their number (copies at most cap of them) */
KPX_API int32_t kpx_sched_tokens(const kpx_sched* s, int32_t request, int32_t* out, int32_t cap);
KPX_API int kpx_sched_forget(kpx_sched* s, int32_t request);
KPX_API int32_t kpx_sched_num_waiting(const kpx_sched* s);
KPX_API int32_t kpx_sched_num_running(const kpx_sched* s);
/* out[0..11] = submitted, admitted, finished, prompt_tokens, reused_tokens, prefilled_tokens,
 * decoded_tokens, prefill_steps, decode_steps, admission_stalls, peak_blocks_in_use, gap_tokens */
KPX_API int kpx_sched_stats(const kpx_sched* s, int64_t* out12);

#ifdef __cplusplus
}
#endif
#endif /* KPX_SCHED_H_ */
