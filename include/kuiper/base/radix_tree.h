// base::RadixTree -- compressed trie over int32 token ids that maps token sequences to
// KV-cache spans, with the observable behaviour of the kuiper header of the same name
// (kuiper/include/base/radix_tree.h:104-532): same public types, fields and methods, same
// results for every call sequence, including its corner cases:
//   * total_cached_tokens is the sum of the kv_length arguments of live terminals (the
//     caller's number is trusted even when it differs from tokens.size()); re-inserting
//     an existing terminal never changes it; inserting the empty sequence never changes it;
//   * find_longest_prefix snaps to the last terminal on the path; without one it reports
//     the tokens consumed including a partial edge, the node above that edge, and
//     kv_cache_pos = -1; edge_offset is whatever the walk left there;
//   * add_reference / release_reference act on an exact-length match whether or not that
//     node is terminal; remove and evict_lru clear the terminal flag but never delete or
//     merge nodes; evict_lru only considers terminal leaves with ref_count == 0, oldest
//     first, and subtracts the node's prefix_length (not its kv_length).
// New here: a terminal may carry the physical block ids that hold its KV span
// (KVCacheInfo::block_ids) and the tree tells its owner when such a span is dropped
// (set_block_release_hook), which is how radix-tree prefixes keep pool blocks alive.
// Children are kept in a vector sorted by first token, so traversal order (dump, the
// order of equal-timestamp eviction candidates) is deterministic.
#ifndef KUIPER_INCLUDE_BASE_RADIX_TREE_H_
#define KUIPER_INCLUDE_BASE_RADIX_TREE_H_

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <utility>
#include <vector>

namespace base {

struct RadixNode;

// Sorted association first-token -> child with the subset of the map interface the tree needs.
class RadixChildren {
 public:
  using Entry = std::pair<int32_t, std::shared_ptr<RadixNode>>;
  bool empty() const { return items_.empty(); }
  size_t size() const { return items_.size(); }
  std::vector<Entry>::const_iterator begin() const { return items_.begin(); }
  std::vector<Entry>::const_iterator end() const { return items_.end(); }
  std::shared_ptr<RadixNode> get(int32_t token) const {
    auto it = lower(token);
    return (it != items_.end() && it->first == token) ? it->second : nullptr;
  }
  void put(int32_t token, std::shared_ptr<RadixNode> node) {
    auto it = lower(token);
    if (it != items_.end() && it->first == token) {
      it->second = std::move(node);
    } else {
      items_.insert(it, Entry(token, std::move(node)));
    }
  }

 private:
  std::vector<Entry>::iterator lower(int32_t token) {
    return std::lower_bound(items_.begin(), items_.end(), token,
                            [](const Entry& e, int32_t t) { return e.first < t; });
  }
  std::vector<Entry>::const_iterator lower(int32_t token) const {
    return std::lower_bound(items_.begin(), items_.end(), token,
                            [](const Entry& e, int32_t t) { return e.first < t; });
  }
  std::vector<Entry> items_;
};

struct RadixNode {
  std::vector<int32_t> edge_tokens;  // tokens on the edge from the parent to this node
  RadixChildren children;
  bool is_terminal = false;
  struct KVCacheInfo {
    int32_t kv_start_pos = 0;
    int32_t kv_length = 0;
    int64_t last_access_time = 0;  // steady-clock milliseconds
    int32_t ref_count = 0;
    std::vector<int32_t> block_ids;  // pool blocks holding [kv_start_pos, kv_start_pos+kv_length)
  } kv_info;
  int32_t prefix_length = 0;  // tokens from the root to this node
  std::weak_ptr<RadixNode> parent;

  RadixNode() = default;
  explicit RadixNode(const std::vector<int32_t>& tokens) : edge_tokens(tokens) {}
  bool is_leaf() const { return children.empty(); }
};

struct RadixMatchResult {
  int32_t matched_length = 0;
  std::shared_ptr<RadixNode> matched_node;
  int32_t edge_offset = 0;
  int32_t kv_cache_pos = -1;
  bool has_kv_cache() const { return kv_cache_pos >= 0 && matched_length > 0; }
};

class RadixTree {
 public:
  using BlockReleaseHook = std::function<void(const std::vector<int32_t>&)>;

  struct Stats {
    int64_t total_nodes = 0;
    int64_t terminal_nodes = 0;
    int64_t total_cached_tokens = 0;
    int32_t max_depth = 0;
  };

  RadixTree() { reset_root(); }

  void insert(const std::vector<int32_t>& tokens, int32_t kv_start_pos, int32_t kv_length) {
    insert(tokens, kv_start_pos, kv_length, std::vector<int32_t>());
  }
  // Same, and the terminal remembers which pool blocks hold the span.
  void insert(const std::vector<int32_t>& tokens, int32_t kv_start_pos, int32_t kv_length,
              const std::vector<int32_t>& block_ids) {
    std::lock_guard<std::mutex> guard(mutex_);
    std::shared_ptr<RadixNode> node = materialise(tokens);
    if (!tokens.empty() && !node->is_terminal) total_cached_tokens_ += kv_length;
    mark_terminal(node, kv_start_pos, kv_length, block_ids);
  }

  RadixMatchResult find_longest_prefix(const std::vector<int32_t>& tokens) const {
    std::lock_guard<std::mutex> guard(mutex_);
    return walk(tokens);
  }

  bool contains(const std::vector<int32_t>& tokens) const {
    std::lock_guard<std::mutex> guard(mutex_);
    RadixMatchResult r = walk(tokens);
    return exact(r, tokens) && r.matched_node->is_terminal;
  }

  bool remove(const std::vector<int32_t>& tokens) {
    std::lock_guard<std::mutex> guard(mutex_);
    RadixMatchResult r = walk(tokens);
    if (!exact(r, tokens) || !r.matched_node->is_terminal) return false;
    total_cached_tokens_ -= r.matched_node->kv_info.kv_length;
    drop_terminal(r.matched_node);
    return true;
  }

  void add_reference(const std::vector<int32_t>& tokens) {
    std::lock_guard<std::mutex> guard(mutex_);
    RadixMatchResult r = walk(tokens);
    if (!exact(r, tokens)) return;
    r.matched_node->kv_info.ref_count += 1;
    r.matched_node->kv_info.last_access_time = now_ms();
  }

  void release_reference(const std::vector<int32_t>& tokens) {
    std::lock_guard<std::mutex> guard(mutex_);
    RadixMatchResult r = walk(tokens);
    if (exact(r, tokens) && r.matched_node->kv_info.ref_count > 0)
      r.matched_node->kv_info.ref_count -= 1;
  }

  void clear() {
    std::lock_guard<std::mutex> guard(mutex_);
    if (release_hook_) release_subtree(root_);
    reset_root();
    total_cached_tokens_ = 0;
  }

  int64_t get_total_cached_tokens() const { return total_cached_tokens_.load(); }

  // Drops unreferenced terminal leaves, least recently used first, until at most
  // max_tokens stay accounted.  Returns the tokens freed (by prefix_length).
  int64_t evict_lru(int64_t max_tokens) {
    std::lock_guard<std::mutex> guard(mutex_);
    if (total_cached_tokens_ <= max_tokens) return 0;
    std::vector<std::shared_ptr<RadixNode>> leaves;
    gather_terminal_leaves(root_, &leaves);
    std::stable_sort(leaves.begin(), leaves.end(),
                     [](const std::shared_ptr<RadixNode>& a, const std::shared_ptr<RadixNode>& b) {
                       return a->kv_info.last_access_time < b->kv_info.last_access_time;
                     });
    int64_t freed = 0;
    for (const auto& leaf : leaves) {
      if (total_cached_tokens_ <= max_tokens) break;
      if (leaf->kv_info.ref_count > 0) continue;
      const int64_t span = leaf->prefix_length;
      drop_terminal(leaf);
      total_cached_tokens_ -= span;
      freed += span;
    }
    return freed;
  }

  // Block-aware reclamation for an allocator under pressure (no counterpart in the reference,
  // whose eviction above only trims a token count): drops unreferenced terminals that hold pool
  // blocks, least recently used first, one at a time, until `enough()` answers true or none is
  // left.  Unlike evict_lru it also takes terminals that have children: every terminal holds
  // its own references on the blocks of its span, so dropping a parent never takes blocks away
  // from a longer registered sequence below it, and spans that only ever gain children (a
  // shared system prompt, earlier turns of a conversation) stay reclaimable.  Returns the
  // kv_length total of what was dropped.
  int64_t reclaim_blocks(const std::function<bool()>& enough) {
    std::lock_guard<std::mutex> guard(mutex_);
    if (enough()) return 0;
    std::vector<std::shared_ptr<RadixNode>> holders;
    gather_block_holders(root_, &holders);
    std::stable_sort(holders.begin(), holders.end(),
                     [](const std::shared_ptr<RadixNode>& a, const std::shared_ptr<RadixNode>& b) {
                       return a->kv_info.last_access_time < b->kv_info.last_access_time;
                     });
    int64_t freed = 0;
    for (const auto& node : holders) {
      if (enough()) break;
      const int64_t span = node->kv_info.kv_length;
      drop_terminal(node);
      total_cached_tokens_ -= span;
      freed += span;
    }
    return freed;
  }

  std::string dump() const {
    std::lock_guard<std::mutex> guard(mutex_);
    std::stringstream out;
    out << "ROOT\n";
    for (const auto& kv : root_->children) print_node(kv.second, "  ", out);
    return out.str();
  }

  Stats get_stats() const {
    std::lock_guard<std::mutex> guard(mutex_);
    Stats s;
    s.total_cached_tokens = total_cached_tokens_;
    // explicit stack: (node, depth)
    std::vector<std::pair<const RadixNode*, int32_t>> todo;
    todo.emplace_back(root_.get(), 0);
    while (!todo.empty()) {
      auto [node, depth] = todo.back();
      todo.pop_back();
      s.total_nodes += 1;
      if (node->is_terminal) s.terminal_nodes += 1;
      if (depth > s.max_depth) s.max_depth = depth;
      for (const auto& kv : node->children) todo.emplace_back(kv.second.get(), depth + 1);
    }
    return s;
  }

  // Called (under the tree's lock) with the block ids of a terminal whose KV span is
  // dropped by remove / evict_lru / clear / being overwritten by a new insert.
  void set_block_release_hook(BlockReleaseHook hook) {
    std::lock_guard<std::mutex> guard(mutex_);
    release_hook_ = std::move(hook);
  }

  // Longest terminal prefix together with the block ids it carries (empty if none).
  RadixMatchResult find_longest_prefix(const std::vector<int32_t>& tokens,
                                       std::vector<int32_t>* block_ids) const {
    std::lock_guard<std::mutex> guard(mutex_);
    RadixMatchResult r = walk(tokens);
    if (block_ids) {
      block_ids->clear();
      if (r.matched_node && r.matched_node->is_terminal && r.kv_cache_pos >= 0)
        *block_ids = r.matched_node->kv_info.block_ids;
    }
    return r;
  }

 private:
  static int64_t now_ms() {
    return std::chrono::duration_cast<std::chrono::milliseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
  }
  static bool exact(const RadixMatchResult& r, const std::vector<int32_t>& tokens) {
    return r.matched_node && r.matched_length == static_cast<int32_t>(tokens.size());
  }
  static size_t common_prefix(const std::vector<int32_t>& edge, const std::vector<int32_t>& tokens,
                              size_t from) {
    const size_t limit = std::min(edge.size(), tokens.size() - from);
    size_t n = 0;
    while (n < limit && edge[n] == tokens[from + n]) ++n;
    return n;
  }
  void reset_root() {
    root_ = std::make_shared<RadixNode>();
    root_->prefix_length = 0;
  }

  // Returns the node that spells `tokens` exactly, creating a leaf or splitting an edge
  // when the tree does not have it yet.
  std::shared_ptr<RadixNode> materialise(const std::vector<int32_t>& tokens) {
    std::shared_ptr<RadixNode> at = root_;
    size_t used = 0;
    while (used < tokens.size()) {
      std::shared_ptr<RadixNode> next = at->children.get(tokens[used]);
      if (!next) {
        auto leaf = std::make_shared<RadixNode>();
        leaf->edge_tokens.assign(tokens.begin() + static_cast<std::ptrdiff_t>(used), tokens.end());
        leaf->prefix_length = static_cast<int32_t>(tokens.size());
        leaf->parent = at;
        at->children.put(tokens[used], leaf);
        return leaf;
      }
      const size_t same = common_prefix(next->edge_tokens, tokens, used);
      if (same == next->edge_tokens.size()) {
        used += same;
        at = next;
        continue;
      }
      // the edge forks after `same` tokens: put a junction there
      auto junction = std::make_shared<RadixNode>();
      junction->edge_tokens.assign(next->edge_tokens.begin(),
                                   next->edge_tokens.begin() + static_cast<std::ptrdiff_t>(same));
      junction->prefix_length = at->prefix_length + static_cast<int32_t>(same);
      junction->parent = at;
      next->edge_tokens.erase(next->edge_tokens.begin(),
                              next->edge_tokens.begin() + static_cast<std::ptrdiff_t>(same));
      next->parent = junction;
      junction->children.put(next->edge_tokens.front(), next);
      at->children.put(tokens[used], junction);
      used += same;
      if (used == tokens.size()) return junction;
      auto leaf = std::make_shared<RadixNode>();
      leaf->edge_tokens.assign(tokens.begin() + static_cast<std::ptrdiff_t>(used), tokens.end());
      leaf->prefix_length = static_cast<int32_t>(tokens.size());
      leaf->parent = junction;
      junction->children.put(leaf->edge_tokens.front(), leaf);
      return leaf;
    }
    return at;
  }

  void mark_terminal(const std::shared_ptr<RadixNode>& node, int32_t start, int32_t length,
                     const std::vector<int32_t>& block_ids) {
    if (node->is_terminal && release_hook_ && !node->kv_info.block_ids.empty())
      release_hook_(node->kv_info.block_ids);
    node->is_terminal = true;
    node->kv_info.kv_start_pos = start;
    node->kv_info.kv_length = length;
    node->kv_info.last_access_time = now_ms();
    node->kv_info.block_ids = block_ids;
  }

  void drop_terminal(const std::shared_ptr<RadixNode>& node) {
    if (release_hook_ && !node->kv_info.block_ids.empty()) release_hook_(node->kv_info.block_ids);
    node->is_terminal = false;
    node->kv_info = RadixNode::KVCacheInfo{};
  }

  RadixMatchResult walk(const std::vector<int32_t>& tokens) const {
    RadixMatchResult r;
    std::shared_ptr<RadixNode> at = root_;
    std::shared_ptr<RadixNode> best = root_->is_terminal ? root_ : nullptr;
    int32_t best_len = 0;
    size_t used = 0;
    while (used < tokens.size()) {
      std::shared_ptr<RadixNode> next = at->children.get(tokens[used]);
      if (!next) break;
      const size_t same = common_prefix(next->edge_tokens, tokens, used);
      used += same;
      if (same < next->edge_tokens.size()) {
        r.edge_offset = static_cast<int32_t>(same);
        break;
      }
      at = next;
      if (at->is_terminal) {
        best = at;
        best_len = static_cast<int32_t>(used);
      }
    }
    if (best) {
      r.matched_node = best;
      r.matched_length = best_len;
      r.kv_cache_pos = best->kv_info.kv_start_pos;
    } else {
      r.matched_node = at;
      r.matched_length = static_cast<int32_t>(used);
    }
    return r;
  }

  void gather_terminal_leaves(const std::shared_ptr<RadixNode>& node,
                              std::vector<std::shared_ptr<RadixNode>>* out) const {
    if (node->is_terminal && node->is_leaf()) out->push_back(node);
    for (const auto& kv : node->children) gather_terminal_leaves(kv.second, out);
  }

  void gather_block_holders(const std::shared_ptr<RadixNode>& node,
                            std::vector<std::shared_ptr<RadixNode>>* out) const {
    if (node->is_terminal && node->kv_info.ref_count == 0 && !node->kv_info.block_ids.empty())
      out->push_back(node);
    for (const auto& kv : node->children) gather_block_holders(kv.second, out);
  }

  void release_subtree(const std::shared_ptr<RadixNode>& node) {
    if (node->is_terminal && !node->kv_info.block_ids.empty()) release_hook_(node->kv_info.block_ids);
    for (const auto& kv : node->children) release_subtree(kv.second);
  }

  void print_node(const std::shared_ptr<RadixNode>& node, const std::string& indent,
                  std::stringstream& out) const {
    out << indent << "Edge[";
    const size_t shown = std::min<size_t>(node->edge_tokens.size(), 5);
    for (size_t i = 0; i < shown; ++i) out << (i ? "," : "") << node->edge_tokens[i];
    if (node->edge_tokens.size() > shown) out << "...+" << (node->edge_tokens.size() - shown);
    out << "]";
    if (node->is_terminal)
      out << " *KV(pos=" << node->kv_info.kv_start_pos << ",len=" << node->kv_info.kv_length
          << ",ref=" << node->kv_info.ref_count << ")";
    out << "\n";
    for (const auto& kv : node->children) print_node(kv.second, indent + "  ", out);
  }

  std::shared_ptr<RadixNode> root_;
  mutable std::mutex mutex_;
  std::atomic<int64_t> total_cached_tokens_{0};
  BlockReleaseHook release_hook_;
};

}  // namespace base
#endif  // KUIPER_INCLUDE_BASE_RADIX_TREE_H_
