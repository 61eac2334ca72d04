// C ABI of the request scheduler (include/kpx_sched.h) over base::KVScheduler.
#include <cstring>
#include <memory>
#include <unordered_set>
#include <vector>

#include "base/kv_scheduler.h"
#include "kpx_sched.h"
#include "kvm_handle.h"

struct kpx_sched {
  kpx_kvm* kvm = nullptr;
  base::KVScheduler* sched = nullptr;
  base::PrefillStep prefill;
  base::DecodeStep decode;
  ~kpx_sched() { delete sched; }
};

namespace {
template <typename T>
void copy_out(T* dst, const std::vector<T>& src) {
  if (dst && !src.empty()) std::memcpy(dst, src.data(), src.size() * sizeof(T));
}
}  // namespace

extern "C" kpx_sched* kpx_sched_create(kpx_kvm* kvm, int32_t prefill_chunk, int32_t max_prefill_tokens,
                                       int32_t max_prefill_rows, int32_t max_decode_batch,
                                       int32_t use_prefix_cache) {
  if (!kvm || prefill_chunk <= 0 || max_prefill_tokens <= 0 || max_prefill_rows <= 0 || max_decode_batch <= 0)
    return nullptr;
  base::KVSchedulerConfig c;
  c.prefill_chunk = prefill_chunk;
  c.max_prefill_tokens = max_prefill_tokens;
  c.max_prefill_rows = max_prefill_rows;
  c.max_decode_batch = max_decode_batch;
  c.use_prefix_cache = use_prefix_cache != 0;
  auto* s = new kpx_sched();
  s->kvm = kvm;
  s->sched = new base::KVScheduler(kvm->pool.get(), kvm->cache.get(), c);
  return s;
}
extern "C" void kpx_sched_destroy(kpx_sched* s) { delete s; }

extern "C" int32_t kpx_sched_submit(kpx_sched* s, const int32_t* prompt, int32_t prompt_len, int32_t max_new_tokens,
                                    int32_t also_register) {
  if (!s || !prompt || prompt_len <= 0) return -1;
  return s->sched->submit(std::vector<int32_t>(prompt, prompt + prompt_len), max_new_tokens, also_register);
}
extern "C" int32_t kpx_sched_submit_turn(kpx_sched* s, const int32_t* prompt, int32_t prompt_len,
                                         int32_t max_new_tokens, int32_t also_register,
                                         const int32_t* turn_suffix, int32_t suffix_len) {
  if (!s || !prompt || prompt_len <= 0 || suffix_len < 0 || (suffix_len > 0 && !turn_suffix)) return -1;
  return s->sched->submit_turn(std::vector<int32_t>(prompt, prompt + prompt_len), max_new_tokens,
                               std::vector<int32_t>(turn_suffix, turn_suffix + suffix_len), also_register);
}
extern "C" int kpx_sched_set_end_tokens(kpx_sched* s, const int32_t* token_ids, int32_t n) {
  if (!s || n < 0 || (n > 0 && !token_ids)) return KPX_ERR_INVALID_ARGUMENT;
  if (n == 0) {
    s->sched->set_end_token_test(nullptr);
    return KPX_OK;
  }
  auto ids = std::make_shared<std::unordered_set<int32_t>>(token_ids, token_ids + n);
  s->sched->set_end_token_test([ids](int32_t t) { return ids->count(t) != 0; });
  return KPX_OK;
}
extern "C" int32_t kpx_sched_admit(kpx_sched* s) { return s ? s->sched->admit() : -1; }

extern "C" int kpx_sched_next_prefill(kpx_sched* s) { return (s && s->sched->next_prefill(&s->prefill)) ? 1 : 0; }
extern "C" int kpx_sched_prefill_shape(const kpx_sched* s, int32_t* rows, int32_t* tokens, int32_t* max_blocks) {
  if (!s) return KPX_ERR_INVALID_ARGUMENT;
  if (rows) *rows = s->prefill.num_rows();
  if (tokens) *tokens = s->prefill.num_tokens();
  if (max_blocks) *max_blocks = s->sched->max_blocks_of(s->prefill.request_ids);
  return KPX_OK;
}
extern "C" int kpx_sched_prefill_arrays(const kpx_sched* s, int32_t* request_ids, int32_t* cu_q_lens,
                                        int32_t* start_pos, int32_t* positions, int64_t* slot_mapping,
                                        int32_t* token_ids, int32_t* completes, int32_t* block_table,
                                        int32_t max_blocks) {
  if (!s) return KPX_ERR_INVALID_ARGUMENT;
  const base::PrefillStep& p = s->prefill;
  copy_out(request_ids, p.request_ids);
  copy_out(cu_q_lens, p.cu_q_lens);
  copy_out(start_pos, p.start_pos);
  copy_out(positions, p.positions);
  copy_out(slot_mapping, p.slot_mapping);
  copy_out(token_ids, p.token_ids);
  copy_out(completes, p.completes);
  if (block_table) return s->sched->fill_block_table(p.request_ids, block_table, max_blocks).get_err_code();
  return KPX_OK;
}
extern "C" int kpx_sched_complete_prefill(kpx_sched* s, const int32_t* sampled, int32_t rows) {
  if (!s || rows != s->prefill.num_rows() || (rows > 0 && !sampled)) return KPX_ERR_INVALID_ARGUMENT;
  s->sched->complete_prefill(s->prefill, std::vector<int32_t>(sampled, sampled + rows));
  s->prefill = base::PrefillStep{};
  return KPX_OK;
}

extern "C" int kpx_sched_next_decode(kpx_sched* s) { return (s && s->sched->next_decode(&s->decode)) ? 1 : 0; }
extern "C" int kpx_sched_decode_shape(const kpx_sched* s, int32_t* rows, int32_t* max_blocks) {
  if (!s) return KPX_ERR_INVALID_ARGUMENT;
  if (rows) *rows = s->decode.num_rows();
  if (max_blocks) *max_blocks = s->sched->max_blocks_of(s->decode.request_ids);
  return KPX_OK;
}
extern "C" int kpx_sched_decode_arrays(const kpx_sched* s, int32_t* request_ids, int32_t* seq_lens,
                                       int32_t* positions, int64_t* slot_mapping, int32_t* token_ids,
                                       int32_t* block_table, int32_t max_blocks) {
  if (!s) return KPX_ERR_INVALID_ARGUMENT;
  const base::DecodeStep& d = s->decode;
  copy_out(request_ids, d.request_ids);
  copy_out(seq_lens, d.seq_lens);
  copy_out(positions, d.positions);
  copy_out(slot_mapping, d.slot_mapping);
  copy_out(token_ids, d.token_ids);
  if (block_table) return s->sched->fill_block_table(d.request_ids, block_table, max_blocks).get_err_code();
  return KPX_OK;
}
extern "C" int kpx_sched_complete_decode(kpx_sched* s, const int32_t* sampled, int32_t rows) {
  if (!s || rows != s->decode.num_rows() || (rows > 0 && !sampled)) return KPX_ERR_INVALID_ARGUMENT;
  s->sched->complete_decode(s->decode, std::vector<int32_t>(sampled, sampled + rows));
  s->decode = base::DecodeStep{};
  return KPX_OK;
}

extern "C" int32_t kpx_sched_state(const kpx_sched* s, int32_t request) {
  return s ? static_cast<int32_t>(s->sched->state(request)) : 3;
}
extern "C" int32_t kpx_sched_reused_tokens(const kpx_sched* s, int32_t request) {
  return s ? s->sched->reused_tokens(request) : -1;
}
extern "C" int32_t kpx_sched_tokens(const kpx_sched* s, int32_t request, int32_t* out, int32_t cap) {
  if (!s) return -1;
  const std::vector<int32_t>* t = s->sched->tokens(request);
  if (!t) return -1;
  const int32_t n = static_cast<int32_t>(t->size());
  if (out && cap > 0) std::memcpy(out, t->data(), sizeof(int32_t) * static_cast<size_t>(n < cap ? n : cap));
  return n;
}
extern "C" int kpx_sched_forget(kpx_sched* s, int32_t request) {
  if (!s) return KPX_ERR_INVALID_ARGUMENT;
  s->sched->forget(request);
  return KPX_OK;
}
extern "C" int32_t kpx_sched_num_waiting(const kpx_sched* s) { return s ? s->sched->num_waiting() : -1; }
extern "C" int32_t kpx_sched_num_running(const kpx_sched* s) { return s ? s->sched->num_running() : -1; }
extern "C" int kpx_sched_stats(const kpx_sched* s, int64_t* out12) {
  if (!s || !out12) return KPX_ERR_INVALID_ARGUMENT;
  const base::KVSchedulerStats& st = s->sched->stats();
  const int64_t v[12] = {st.submitted, st.admitted, st.finished, st.prompt_tokens, st.reused_tokens,
                         st.prefilled_tokens, st.decoded_tokens, st.prefill_steps, st.decode_steps,
                         st.admission_stalls, st.peak_blocks_in_use, st.gap_tokens};
  std::memcpy(out12, v, sizeof(v));
  return KPX_OK;
}
