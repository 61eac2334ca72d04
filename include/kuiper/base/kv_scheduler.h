// Request scheduler over the paged KV cache: turns many concurrent requests into the work
// lists the kernels take (slot mappings, block tables, lengths), with prefix reuse.
//
// Per request it follows the order of operations of the reference's generate_response
// (demo/inference_common.h:1050-1262) and PrefixCacheManager (:757-853):
//     match (adds a reference)  ->  prefill from the matched position, in chunks  ->
//     one decode step per generated token  ->  (fill the gap)  ->  register the sequence  ->
//     release the match.
// "Fill the gap" is the reference's end-of-turn fix-up (demo/inference_common.h:1334-1358): the
// last sampled token (the end marker) was never fed in, and the chat template appends
// separator tokens after it, so the history that the next turn will present is longer than
// what the cache holds; the missing tokens are prefilled, without sampling, before the
// whole history is registered.  A request asks for it with submit_turn().
// The reference runs one request at a time on a contiguous cache; here requests run
// concurrently on the block pool: a hit maps the matched blocks by reference, a sequence that
// appends into a shared, partly filled block first gets a private copy (copy-on-write, logged
// by PagedKVManager for the device), and admission is gated by free blocks so that a running
// request can never run out of blocks (the reference's only guard is the
// "context length exceeded" check at :1066-1074).
// Differences from the reference, on purpose:
//   * a full hit still recomputes the last prompt token, so that there is an attention output
//     to sample from (the reference skips prefill and reads a stale logits buffer);
//   * without the gap fill, the registered sequence is cut to the tokens whose K/V are in the
//     cache (the last sampled token has none yet).
#ifndef KUIPER_INCLUDE_BASE_KV_SCHEDULER_H_
#define KUIPER_INCLUDE_BASE_KV_SCHEDULER_H_

#include <cstdint>
#include <algorithm>
#include <deque>
#include <functional>
#include <unordered_map>
#include <vector>

#include "paged_kv.h"
#include "prefix_cache.h"

namespace base {

struct KVSchedulerConfig {
  int32_t prefill_chunk = 512;         // most tokens of one request in one prefill step
  int32_t max_prefill_tokens = 2048;   // most tokens of all requests in one prefill step
  int32_t max_prefill_rows = 64;       // most requests in one prefill step
  int32_t max_decode_batch = 256;      // most requests in one decode step
  bool use_prefix_cache = true;
};

enum class RequestState : int32_t { kWaiting = 0, kPrefill = 1, kDecode = 2, kFinished = 3, kGapFill = 4 };

// Inputs of one kpx_rope_append / kpx_append + kpx_paged_prefill call sequence.
struct PrefillStep {
  std::vector<int32_t> request_ids;   // one per batch row
  std::vector<int32_t> cu_q_lens;     // [rows + 1] offsets of the rows' tokens
  std::vector<int32_t> start_pos;     // [rows] cache position of each row's first token
  std::vector<int32_t> positions;     // [tokens] cache position (RoPE position) of every token
  std::vector<int64_t> slot_mapping;  // [tokens] pool slot of every token
  std::vector<int32_t> token_ids;     // [tokens] ids to embed
  std::vector<int32_t> completes;     // [rows] 1: the row ends its prompt, a token is sampled from its last output
  int32_t num_tokens() const { return static_cast<int32_t>(positions.size()); }
  int32_t num_rows() const { return static_cast<int32_t>(request_ids.size()); }
};

// Inputs of one decode step (kpx_rope_append with num_tokens = rows, then kpx_paged_decode).
struct DecodeStep {
  std::vector<int32_t> request_ids;   // one per batch row
  std::vector<int32_t> seq_lens;      // [rows] tokens each row attends to (the new one included)
  std::vector<int32_t> positions;     // [rows] cache position of the new token
  std::vector<int64_t> slot_mapping;  // [rows]
  std::vector<int32_t> token_ids;     // [rows] the token fed in (the one sampled last)
  int32_t num_rows() const { return static_cast<int32_t>(request_ids.size()); }
};

struct KVSchedulerStats {
  int64_t submitted = 0, admitted = 0, finished = 0;
  int64_t prompt_tokens = 0, reused_tokens = 0, prefilled_tokens = 0, decoded_tokens = 0;
  int64_t gap_tokens = 0;              // end-of-turn tokens prefilled without sampling
  int64_t prefill_steps = 0, decode_steps = 0;
  int64_t admission_stalls = 0;        // admit() calls that left a request waiting for blocks
  int32_t peak_blocks_in_use = 0;
};

class KVScheduler {
 public:
  // The pool and the cache are owned by the caller (they are also what the device flush and
  // the block-table queries talk to); the cache's block release hook must already point at
  // the pool.
  KVScheduler(PagedKVManager* pool, PrefixCache* cache, const KVSchedulerConfig& config)
      : pool_(pool), cache_(cache), config_(config) {}

  const KVSchedulerConfig& config() const { return config_; }
  const KVSchedulerStats& stats() const { return stats_; }

  // Queues a request; returns its id (ids count up from 0) or -1 on bad arguments, among them a
  // request whose last token could never be cached because the whole pool is too small for it
  // (it would otherwise wait at the head of the queue for ever).
  // also_register > 0: when the request finishes, its first also_register tokens are
  // registered as a prefix of their own as well (a shared system prompt: the tree only
  // reports a hit at a registered length, radix_tree.h:375-449).
  int32_t submit(const std::vector<int32_t>& prompt, int32_t max_new_tokens, int32_t also_register = 0) {
    if (prompt.empty() || max_new_tokens < 1 || also_register < 0) return -1;
    if (blocks_for(static_cast<int32_t>(prompt.size()) + max_new_tokens - 1) > pool_->config().num_blocks) return -1;
    const int32_t id = next_id_++;
    Request& r = requests_[id];
    r.tokens = prompt;
    r.prompt_len = static_cast<int32_t>(prompt.size());
    r.max_new = max_new_tokens;
    r.also_register = also_register;
    waiting_.push_back(id);
    ++stats_.submitted;
    stats_.prompt_tokens += r.prompt_len;
    return id;
  }

  // A request that is one turn of a conversation: when generation ends, the last sampled token
  // and `turn_suffix` (the template's separators after it; may be empty) are prefilled too, so
  // that the registered sequence is the whole history the next turn starts with.
  int32_t submit_turn(const std::vector<int32_t>& prompt, int32_t max_new_tokens,
                      const std::vector<int32_t>& turn_suffix, int32_t also_register = 0) {
    if (prompt.empty() || max_new_tokens < 1) return -1;
    // with the gap fill the history grows by the last sampled token and the suffix
    const int64_t final_tokens = static_cast<int64_t>(prompt.size()) + max_new_tokens + static_cast<int64_t>(turn_suffix.size());
    if (final_tokens > static_cast<int64_t>(pool_->config().num_blocks) * pool_->config().block_size) return -1;
    const int32_t id = submit(prompt, max_new_tokens, also_register);
    if (id < 0) return id;
    Request& r = requests_[id];
    r.fill_gap = true;
    r.turn_suffix = turn_suffix;
    return id;
  }

  // Moves waiting requests into the running set, first come first served, while the pool can
  // hold each one to its last token.  Returns how many were admitted.
  int32_t admit() {
    int32_t n = 0;
    while (!waiting_.empty()) {
      const int32_t id = waiting_.front();
      if (!try_admit(id)) {
        ++stats_.admission_stalls;
        break;
      }
      waiting_.pop_front();
      running_.push_back(id);
      ++stats_.admitted;
      ++n;
    }
    return n;
  }

  // Next prefill step: running requests with prompt tokens left, oldest first.  False when
  // there is nothing to prefill.
  bool next_prefill(PrefillStep* step) {
    *step = PrefillStep{};
    step->cu_q_lens.push_back(0);
    int32_t budget = config_.max_prefill_tokens;
    for (int32_t id : running_) {
      Request& r = requests_[id];
      if (r.state != RequestState::kPrefill && r.state != RequestState::kGapFill) continue;
      if (budget <= 0 || step->num_rows() >= config_.max_prefill_rows) break;
      const bool gap = r.state == RequestState::kGapFill;
      const int32_t target = gap ? static_cast<int32_t>(r.tokens.size()) : r.prompt_len;
      const int32_t n = std::min({config_.prefill_chunk, target - r.computed, budget});
      if (n <= 0) continue;
      std::vector<int64_t> slots;
      if (!pool_->append(r.seq, n, &slots)) continue;  // cannot happen after admission; skip, never corrupt
      step->request_ids.push_back(id);
      step->start_pos.push_back(r.computed);
      for (int32_t i = 0; i < n; ++i) {
        step->positions.push_back(r.computed + i);
        step->token_ids.push_back(r.tokens[static_cast<size_t>(r.computed + i)]);
        step->slot_mapping.push_back(slots[static_cast<size_t>(i)]);
      }
      step->cu_q_lens.push_back(step->num_tokens());
      r.computed += n;
      step->completes.push_back(!gap && r.computed == r.prompt_len ? 1 : 0);
      budget -= n;
      stats_.prefilled_tokens += n;
      if (gap) stats_.gap_tokens += n;
    }
    note_usage();
    if (step->num_rows() == 0) return false;
    ++stats_.prefill_steps;
    return true;
  }

  // The tokens sampled for the rows of `step` that completed their prompt (one entry per row;
  // entries of rows that did not complete are ignored).
  void complete_prefill(const PrefillStep& step, const std::vector<int32_t>& sampled) {
    for (int32_t i = 0; i < step.num_rows(); ++i) {
      Request& r = requests_[step.request_ids[static_cast<size_t>(i)]];
      // a gap row whose history is now cached in full is done (nothing is sampled from it)
      if (r.state == RequestState::kGapFill && r.computed == static_cast<int32_t>(r.tokens.size()))
        r.state = RequestState::kFinished;
      if (!step.completes[static_cast<size_t>(i)]) continue;
      r.state = RequestState::kDecode;
      push_token(step.request_ids[static_cast<size_t>(i)], r, sampled[static_cast<size_t>(i)]);
    }
    sweep_finished();
  }

  // Next decode step: every running request that has a sampled token to feed in.
  bool next_decode(DecodeStep* step) {
    *step = DecodeStep{};
    for (int32_t id : running_) {
      Request& r = requests_[id];
      if (r.state != RequestState::kDecode) continue;
      if (step->num_rows() >= config_.max_decode_batch) break;
      std::vector<int64_t> slots;
      if (!pool_->append(r.seq, 1, &slots)) continue;
      step->request_ids.push_back(id);
      step->positions.push_back(r.computed);
      step->slot_mapping.push_back(slots[0]);
      step->token_ids.push_back(r.tokens.back());
      r.computed += 1;
      step->seq_lens.push_back(r.computed);
      ++stats_.decoded_tokens;
    }
    note_usage();
    if (step->num_rows() == 0) return false;
    ++stats_.decode_steps;
    return true;
  }

  void complete_decode(const DecodeStep& step, const std::vector<int32_t>& sampled) {
    for (int32_t i = 0; i < step.num_rows(); ++i) {
      const int32_t id = step.request_ids[static_cast<size_t>(i)];
      push_token(id, requests_[id], sampled[static_cast<size_t>(i)]);
    }
    sweep_finished();
  }

  // Optional end-of-sequence test on a sampled token (the reference: model.is_sentence_ending).
  void set_end_token_test(std::function<bool(int32_t)> fn) { is_end_ = std::move(fn); }

  // Block table rows of the given requests: ids then -1 padding.
  Status fill_block_table(const std::vector<int32_t>& request_ids, int32_t* table, int32_t max_blocks) const {
    for (size_t i = 0; i < request_ids.size(); ++i) {
      auto it = requests_.find(request_ids[i]);
      if (it == requests_.end() || it->second.seq < 0) return error::InvalidArgument("request is not running");
      Status st = pool_->fill_block_table_row(it->second.seq, table + i * static_cast<size_t>(max_blocks), max_blocks);
      if (!st) return st;
    }
    return error::Success();
  }
  int32_t max_blocks_of(const std::vector<int32_t>& request_ids) const {
    int32_t m = 0;
    for (int32_t id : request_ids) {
      auto it = requests_.find(id);
      if (it == requests_.end() || it->second.seq < 0) continue;
      const std::vector<int32_t>* b = pool_->blocks(it->second.seq);
      if (b) m = std::max<int32_t>(m, static_cast<int32_t>(b->size()));
    }
    return m;
  }

  RequestState state(int32_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? RequestState::kFinished : it->second.state;
  }
  int32_t reused_tokens(int32_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? -1 : it->second.reused;
  }
  // prompt followed by the tokens generated so far (and, once a turn has ended, its suffix)
  const std::vector<int32_t>* tokens(int32_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? nullptr : &it->second.tokens;
  }
  int32_t num_waiting() const { return static_cast<int32_t>(waiting_.size()); }
  int32_t num_running() const { return static_cast<int32_t>(running_.size()); }
  bool idle() const { return waiting_.empty() && running_.empty(); }
  // Forget a finished request (its token list is kept until then for the caller to read).
  void forget(int32_t id) {
    auto it = requests_.find(id);
    if (it != requests_.end() && it->second.state == RequestState::kFinished) requests_.erase(it);
  }

 private:
  struct Request {
    std::vector<int32_t> tokens;  // prompt + generated
    int32_t prompt_len = 0, max_new = 0;
    int32_t seq = -1;             // pool sequence while running
    int32_t reused = 0;           // tokens served by the prefix cache
    int32_t computed = 0;         // tokens whose K/V are in the cache
    int32_t reserved = 0;         // blocks this request may still take from the free list
    int32_t also_register = 0;    // extra prefix length to register at the end
    bool fill_gap = false;        // prefill the end-of-turn tokens before registering
    std::vector<int32_t> turn_suffix;
    std::vector<int32_t> matched_prefix;
    RequestState state = RequestState::kWaiting;
  };

  int32_t blocks_for(int32_t tokens) const {
    const int32_t bs = pool_->config().block_size;
    return (tokens + bs - 1) / bs;
  }
  // Most tokens the request will ever have in the cache: the last sampled token is cached only
  // by the gap fill, which also adds the turn's suffix.
  static int32_t final_len(const Request& r) {
    const int32_t n = r.prompt_len + r.max_new - 1;
    return r.fill_gap ? n + 1 + static_cast<int32_t>(r.turn_suffix.size()) : n;
  }

  bool try_admit(int32_t id) {
    Request& r = requests_[id];
    const int32_t seq = pool_->add_sequence();
    int32_t reused = 0;
    std::vector<int32_t> matched;
    if (config_.use_prefix_cache && cache_) {
      PrefixMatchResult m = cache_->match(r.tokens);  // nothing generated yet: tokens == prompt
      if (m.cache_hit && m.matched_tokens > 0 && !m.block_ids.empty()) {
        // keep the last prompt token to compute: its output is what the first token is sampled from
        const int32_t use = std::min(m.matched_tokens, r.prompt_len - 1);
        if (use > 0 && pool_->map_prefix(seq, m.block_ids, use)) {
          reused = use;
          matched = m.matched_prefix;
        } else {
          cache_->release(m.matched_prefix);
        }
      } else if (m.cache_hit) {
        cache_->release(m.matched_prefix);
      }
    }
    // Blocks still to come from the free list until the request's last token is cached: the
    // blocks of its final length minus the mapped ones, plus one if the first append lands in
    // a shared, partly filled block (copy-on-write).
    const int32_t bs = pool_->config().block_size;
    const int32_t mapped = blocks_for(reused);
    const int32_t need = blocks_for(final_len(r)) - mapped + ((reused % bs) != 0 ? 1 : 0);
    int32_t avail = pool_->num_free() - reserved_total_;
    if (need > avail && config_.use_prefix_cache && cache_) {
      // Spans nobody references make room, oldest first, and only as many as it takes.  (The
      // cache's evict() would be the wrong tool: its argument is the token count to keep, and
      // its token accounting does not map one to one onto blocks.)
      cache_->reclaim_blocks([&] { return pool_->num_free() - reserved_total_ >= need; });
      avail = pool_->num_free() - reserved_total_;
    }
    if (need > avail) {
      if (!matched.empty()) cache_->release(matched);
      pool_->free_sequence(seq);
      return false;
    }
    r.seq = seq;
    r.reused = reused;
    r.computed = reused;
    r.matched_prefix = std::move(matched);
    r.reserved = need;
    reserved_total_ += need;
    r.state = RequestState::kPrefill;
    stats_.reused_tokens += reused;
    return true;
  }

  void push_token(int32_t id, Request& r, int32_t token) {
    (void)id;
    r.tokens.push_back(token);
    const int32_t generated = static_cast<int32_t>(r.tokens.size()) - r.prompt_len;
    if (generated >= r.max_new || (is_end_ && is_end_(token))) {
      if (r.fill_gap) {
        r.tokens.insert(r.tokens.end(), r.turn_suffix.begin(), r.turn_suffix.end());
        r.state = RequestState::kGapFill;
      } else {
        r.state = RequestState::kFinished;
      }
    }
  }

  // Finished requests: register what is cached, release the match, give the sequence back.
  void sweep_finished() {
    for (size_t i = 0; i < running_.size();) {
      Request& r = requests_[running_[i]];
      if (r.state != RequestState::kFinished) {
        ++i;
        continue;
      }
      if (config_.use_prefix_cache && cache_ && r.computed > 0) {
        std::vector<int32_t> cached(r.tokens.begin(), r.tokens.begin() + r.computed);
        std::vector<int32_t> blocks = pool_->prefix_blocks(r.seq, r.computed);
        if (pool_->retain(blocks)) cache_->insert(cached, 0, r.computed, blocks);
        if (r.also_register > 0 && r.also_register < r.computed) {
          std::vector<int32_t> head(r.tokens.begin(), r.tokens.begin() + r.also_register);
          std::vector<int32_t> head_blocks = pool_->prefix_blocks(r.seq, r.also_register);
          if (pool_->retain(head_blocks)) cache_->insert(head, 0, r.also_register, head_blocks);
        }
      }
      if (!r.matched_prefix.empty()) cache_->release(r.matched_prefix);
      r.matched_prefix.clear();
      pool_->free_sequence(r.seq);
      r.seq = -1;
      reserved_total_ -= r.reserved;
      r.reserved = 0;
      ++stats_.finished;
      running_.erase(running_.begin() + static_cast<std::ptrdiff_t>(i));
    }
  }

  // Blocks taken since the last look reduce what the running requests still hold in reserve.
  void note_usage() {
    int32_t reserve = 0;
    const int32_t bs = pool_->config().block_size;
    for (int32_t id : running_) {
      Request& r = requests_[id];
      if (r.seq < 0) continue;
      const std::vector<int32_t>* b = pool_->blocks(r.seq);
      const int32_t have = b ? static_cast<int32_t>(b->size()) : 0;
      // a copy-on-write still ahead: the sequence has not appended yet and its last block is shared and partial
      const bool cow_ahead = (r.computed == r.reused) && (r.reused % bs) != 0;
      r.reserved = std::max(0, blocks_for(final_len(r)) - have) + (cow_ahead ? 1 : 0);
      reserve += r.reserved;
    }
    reserved_total_ = reserve;
    const int32_t in_use = pool_->config().num_blocks - pool_->num_free();
    stats_.peak_blocks_in_use = std::max(stats_.peak_blocks_in_use, in_use);
  }

  PagedKVManager* pool_;
  PrefixCache* cache_;
  KVSchedulerConfig config_;
  KVSchedulerStats stats_;
  std::unordered_map<int32_t, Request> requests_;
  std::deque<int32_t> waiting_;
  std::vector<int32_t> running_;
  std::function<bool(int32_t)> is_end_;
  int32_t next_id_ = 0;
  int32_t reserved_total_ = 0;
};

}  // namespace base
#endif  // KUIPER_INCLUDE_BASE_KV_SCHEDULER_H_
