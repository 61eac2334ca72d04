// base::PrefixCache -- prefix reuse policy on top of base::RadixTree, with the observable
// behaviour of kuiper/include/base/prefix_cache.h:39-342: same config, result and stats
// types, same counters after every call.  Points a re-implementation has to get right:
//   * match() counts the request and its tokens before looking up, on hits and misses
//     alike; an empty request returns early and counts nothing;
//   * a hit needs a terminal prefix (kv position >= 0) of at least min_prefix_length
//     tokens; a hit takes a reference on that prefix, the caller gives it back with
//     release();
//   * insert() ignores empty sequences and kv_length <= 0 and runs the eviction check
//     BEFORE inserting (usage above the threshold -> evict down to 80 % of capacity), so
//     usage may end above the threshold;
//   * evict() counts one eviction event and the evicted tokens only when something went.
// New here: spans may carry the pool blocks that hold them (insert with block ids), a hit
// reports the blocks covering the matched tokens, and the owner of the block pool can
// learn when a cached span is dropped (set_block_release_hook).
#ifndef KUIPER_INCLUDE_BASE_PREFIX_CACHE_H_
#define KUIPER_INCLUDE_BASE_PREFIX_CACHE_H_

#include <atomic>
#include <cstdint>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "radix_tree.h"

namespace base {

struct PrefixMatchResult {
  int32_t matched_tokens = 0;
  bool cache_hit = false;
  int32_t prefill_start_pos = 0;  // first position the caller still has to prefill
  int32_t prefill_count = 0;
  float reuse_ratio = 0.0f;
  std::vector<int32_t> matched_prefix;  // key to hand back to release()
  std::vector<int32_t> block_ids;       // pool blocks covering the matched tokens (may be empty)
};

// Declared by the reference next to the cache (prefix_cache.h:64-73) and unused there;
// kept so code that names the type still compiles.
struct KVCacheBlock {
  int32_t start_pos = 0;
  int32_t length = 0;
  int32_t ref_count = 0;
  int64_t last_access = 0;
  bool is_valid = false;
  std::vector<int32_t> tokens;
};

struct PrefixCacheConfig {
  int64_t max_cached_tokens = 65536;
  int32_t min_prefix_length = 4;
  bool enable_auto_eviction = true;
  float eviction_threshold = 0.9f;
  bool enable_stats = true;
};

struct PrefixCacheStats {
  std::atomic<int64_t> total_requests{0};
  std::atomic<int64_t> cache_hits{0};
  std::atomic<int64_t> cache_misses{0};
  std::atomic<int64_t> total_tokens_processed{0};
  std::atomic<int64_t> tokens_reused{0};
  std::atomic<int64_t> tokens_computed{0};
  std::atomic<int64_t> eviction_count{0};
  std::atomic<int64_t> tokens_evicted{0};

  void reset() {
    for (std::atomic<int64_t>* c : {&total_requests, &cache_hits, &cache_misses, &total_tokens_processed,
                                    &tokens_reused, &tokens_computed, &eviction_count, &tokens_evicted})
      c->store(0);
  }
  float hit_rate() const { return ratio(cache_hits.load(), total_requests.load()); }
  float reuse_rate() const { return ratio(tokens_reused.load(), total_tokens_processed.load()); }
  std::string to_string() const {
    std::stringstream s;
    s << "PrefixCache Stats:\n"
      << "  Total requests: " << total_requests.load() << "\n"
      << "  Cache hits: " << cache_hits.load() << " (" << (hit_rate() * 100) << "%)\n"
      << "  Cache misses: " << cache_misses.load() << "\n"
      << "  Total tokens: " << total_tokens_processed.load() << "\n"
      << "  Tokens reused: " << tokens_reused.load() << " (" << (reuse_rate() * 100) << "%)\n"
      << "  Tokens computed: " << tokens_computed.load() << "\n"
      << "  Evictions: " << eviction_count.load() << "\n"
      << "  Tokens evicted: " << tokens_evicted.load() << "\n";
    return s.str();
  }

 private:
  static float ratio(int64_t part, int64_t whole) {
    return whole == 0 ? 0.0f : static_cast<float>(part) / whole;
  }
};

class PrefixCache {
 public:
  explicit PrefixCache(const PrefixCacheConfig& config = PrefixCacheConfig())
      : config_(config), tree_(new RadixTree()) {}

  PrefixMatchResult match(const std::vector<int32_t>& tokens) {
    PrefixMatchResult out;
    const int32_t n = static_cast<int32_t>(tokens.size());
    out.prefill_count = n;
    if (n == 0) return out;
    const bool stats = config_.enable_stats;
    if (stats) {
      stats_.total_requests += 1;
      stats_.total_tokens_processed += n;
    }
    std::vector<int32_t> blocks;
    const RadixMatchResult found = tree_->find_longest_prefix(tokens, &blocks);
    const bool hit = found.has_kv_cache() && found.matched_length >= config_.min_prefix_length;
    if (!hit) {
      if (stats) {
        stats_.cache_misses += 1;
        stats_.tokens_computed += n;
      }
      return out;
    }
    const int32_t m = found.matched_length;
    out.cache_hit = true;
    out.matched_tokens = m;
    out.prefill_start_pos = m;
    out.prefill_count = n - m;
    out.reuse_ratio = static_cast<float>(m) / tokens.size();
    out.matched_prefix.assign(tokens.begin(), tokens.begin() + m);
    out.block_ids = std::move(blocks);
    tree_->add_reference(out.matched_prefix);
    if (stats) {
      stats_.cache_hits += 1;
      stats_.tokens_reused += m;
      stats_.tokens_computed += out.prefill_count;
    }
    return out;
  }

  void insert(const std::vector<int32_t>& tokens, int32_t kv_start_pos, int32_t kv_length) {
    insert(tokens, kv_start_pos, kv_length, std::vector<int32_t>());
  }
  void insert(const std::vector<int32_t>& tokens, int32_t kv_start_pos, int32_t kv_length,
              const std::vector<int32_t>& block_ids) {
    if (tokens.empty() || kv_length <= 0) return;
    if (config_.enable_auto_eviction && get_usage_ratio() > config_.eviction_threshold)
      evict(static_cast<int64_t>(config_.max_cached_tokens * 0.8));
    tree_->insert(tokens, kv_start_pos, kv_length, block_ids);
  }

  void release(const std::vector<int32_t>& tokens) {
    if (!tokens.empty()) tree_->release_reference(tokens);
  }
  bool remove(const std::vector<int32_t>& tokens) { return tree_->remove(tokens); }
  void clear() { tree_->clear(); }

  int64_t get_cached_tokens() const { return tree_->get_total_cached_tokens(); }
  float get_usage_ratio() const {
    return static_cast<float>(get_cached_tokens()) / config_.max_cached_tokens;
  }

  int64_t evict(int64_t target_tokens) {
    const int64_t gone = tree_->evict_lru(target_tokens);
    if (gone > 0 && config_.enable_stats) {
      stats_.eviction_count += 1;
      stats_.tokens_evicted += gone;
    }
    return gone;
  }

  // Frees pool blocks for an allocator that is short: unreferenced spans go, oldest first,
  // until `enough()` is true (RadixTree::reclaim_blocks).  Counted like an eviction.
  int64_t reclaim_blocks(const std::function<bool()>& enough) {
    const int64_t gone = tree_->reclaim_blocks(enough);
    if (gone > 0 && config_.enable_stats) {
      stats_.eviction_count += 1;
      stats_.tokens_evicted += gone;
    }
    return gone;
  }

  const PrefixCacheStats& get_stats() const { return stats_; }
  void reset_stats() { stats_.reset(); }
  const PrefixCacheConfig& get_config() const { return config_; }
  void set_config(const PrefixCacheConfig& config) { config_ = config; }
  std::string dump_tree() const { return tree_->dump(); }
  RadixTree::Stats get_tree_stats() const { return tree_->get_stats(); }

  void set_block_release_hook(RadixTree::BlockReleaseHook hook) {
    tree_->set_block_release_hook(std::move(hook));
  }

 private:
  PrefixCacheConfig config_;
  std::unique_ptr<RadixTree> tree_;
  PrefixCacheStats stats_;
};

}  // namespace base
#endif  // KUIPER_INCLUDE_BASE_PREFIX_CACHE_H_
