// Paged KV-cache bookkeeping on the host: block pool with reference counts, per-sequence
// block lists, slot mappings, prefix sharing and copy-on-write of a shared last block.
//
// The reference keeps one contiguous cache per layer and has none of this
// (kuiper/source/model/qwen3.cpp:845-851, model.cpp:348-385); the rules below are the
// specification the CUDA path and its tests are held to:
//   * a pool has num_blocks blocks of block_size token slots; slot = block*block_size + off;
//   * the free list starts as a seeded Fisher-Yates permutation of 0..num_blocks-1 driven
//     by splitmix64(seed) (identity order when shuffle is off); allocation pops its front,
//     a block whose count drops to zero is pushed at its back;
//   * a sequence owns one reference on each of its blocks; a radix-tree span that lists a
//     block owns one more; map_prefix() takes references on ceil(n/block_size) listed blocks;
//   * append(): a token landing in a new block allocates one; a token landing in a partly
//     filled last block whose count is above 1 first replaces it by a private copy
//     (copy-on-write: new block allocated, a (src, dst) copy recorded, one reference on src
//     given back);
//   * an operation that would need more free blocks than there are fails with
//     kOutOfBlocks and changes nothing.
// Every count change and copy is also logged so that the device-side mirrors (the
// refcount array and the pools) can be updated by kpx_refcount_update /
// kpx_cow_copy_blocks: take_pending() hands the log over.
#ifndef KUIPER_INCLUDE_BASE_PAGED_KV_H_
#define KUIPER_INCLUDE_BASE_PAGED_KV_H_

#include <cstdint>
#include <algorithm>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "base.h"

namespace base {

struct PagedKVConfig {
  int32_t block_size = 16;
  int32_t num_blocks = 0;
  uint64_t seed = 0;
  bool shuffle = true;
};

struct BlockCopy {
  int32_t src = -1, dst = -1;
};
struct BlockRefDelta {
  int32_t block = -1, delta = 0;
};

inline uint64_t splitmix64_next(uint64_t* state) {
  uint64_t z = (*state += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

class PagedKVManager {
 public:
  explicit PagedKVManager(const PagedKVConfig& config)
      : config_(config), ref_(static_cast<size_t>(config.num_blocks), 0) {
    std::vector<int32_t> order(static_cast<size_t>(config.num_blocks));
    for (int32_t i = 0; i < config.num_blocks; ++i) order[static_cast<size_t>(i)] = i;
    if (config.shuffle) {
      uint64_t state = config.seed;
      for (int64_t i = config.num_blocks - 1; i > 0; --i) {
        const uint64_t j = splitmix64_next(&state) % static_cast<uint64_t>(i + 1);
        std::swap(order[static_cast<size_t>(i)], order[static_cast<size_t>(j)]);
      }
    }
    free_.assign(order.begin(), order.end());
  }

  const PagedKVConfig& config() const { return config_; }
  int32_t num_free() const { return static_cast<int32_t>(free_.size()); }
  int32_t ref_count(int32_t block) const { return in_range(block) ? ref_[static_cast<size_t>(block)] : -1; }
  const std::vector<int32_t>& ref_counts() const { return ref_; }
  int64_t cow_events() const { return cow_events_; }
  // blocks referenced more than once
  int32_t num_shared() const {
    int32_t n = 0;
    for (int32_t r : ref_) n += r > 1 ? 1 : 0;
    return n;
  }

  int32_t add_sequence() {
    const int32_t id = next_seq_++;
    seqs_[id] = Sequence{};
    return id;
  }
  bool has_sequence(int32_t seq) const { return seqs_.count(seq) != 0; }
  int32_t length(int32_t seq) const {
    auto it = seqs_.find(seq);
    return it == seqs_.end() ? -1 : it->second.length;
  }
  const std::vector<int32_t>* blocks(int32_t seq) const {
    auto it = seqs_.find(seq);
    return it == seqs_.end() ? nullptr : &it->second.blocks;
  }

  // Start a fresh sequence on blocks another owner already filled: the first n_tokens
  // positions are served by block_ids[0 .. ceil(n/bs)-1], shared by reference.
  Status map_prefix(int32_t seq, const std::vector<int32_t>& block_ids, int32_t n_tokens) {
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return error::InvalidArgument("unknown sequence");
    if (it->second.length != 0 || !it->second.blocks.empty())
      return error::InvalidArgument("map_prefix needs an empty sequence");
    if (n_tokens < 0) return error::InvalidArgument("negative prefix length");
    const int32_t need = blocks_for(n_tokens);
    if (static_cast<int32_t>(block_ids.size()) < need)
      return error::InvalidArgument("prefix lists too few blocks");
    for (int32_t i = 0; i < need; ++i) {
      const int32_t b = block_ids[static_cast<size_t>(i)];
      if (!in_range(b) || ref_[static_cast<size_t>(b)] <= 0)
        return error::InvalidArgument("prefix lists a block that is not live");
    }
    for (int32_t i = 0; i < need; ++i) {
      change(block_ids[static_cast<size_t>(i)], +1);
      it->second.blocks.push_back(block_ids[static_cast<size_t>(i)]);
    }
    it->second.length = n_tokens;
    return error::Success();
  }

  // Reserve slots for the next n tokens of the sequence; slots[i] receives the slot of
  // position length+i.  All or nothing.
  Status append(int32_t seq, int32_t n, std::vector<int64_t>* slots) {
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return error::InvalidArgument("unknown sequence");
    if (n < 0) return error::InvalidArgument("negative token count");
    Sequence& s = it->second;
    const int32_t bs = config_.block_size;
    const bool partial_last = (s.length % bs) != 0;
    const bool cow = n > 0 && partial_last && ref_[static_cast<size_t>(s.blocks.back())] > 1;
    const int32_t fresh = blocks_for(s.length + n) - static_cast<int32_t>(s.blocks.size());
    if (fresh + (cow ? 1 : 0) > num_free())
      return error::OutOfBlocks("block pool exhausted");
    if (cow) {
      const int32_t old = s.blocks.back();
      const int32_t mine = take_free();
      copies_.push_back(BlockCopy{old, mine});
      change(old, -1);
      s.blocks.back() = mine;
      ++cow_events_;
    }
    for (int32_t i = 0; i < fresh; ++i) s.blocks.push_back(take_free());
    if (slots) {
      slots->resize(static_cast<size_t>(n));
      for (int32_t i = 0; i < n; ++i) {
        const int32_t pos = s.length + i;
        (*slots)[static_cast<size_t>(i)] =
            static_cast<int64_t>(s.blocks[static_cast<size_t>(pos / bs)]) * bs + pos % bs;
      }
    }
    s.length += n;
    return error::Success();
  }

  Status free_sequence(int32_t seq) {
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return error::InvalidArgument("unknown sequence");
    for (int32_t b : it->second.blocks) change(b, -1);
    seqs_.erase(it);
    return error::Success();
  }

  // Block ids serving the first n_tokens positions of the sequence.
  std::vector<int32_t> prefix_blocks(int32_t seq, int32_t n_tokens) const {
    std::vector<int32_t> out;
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return out;
    const int32_t need = std::min<int32_t>(blocks_for(n_tokens), static_cast<int32_t>(it->second.blocks.size()));
    out.assign(it->second.blocks.begin(), it->second.blocks.begin() + need);
    return out;
  }

  // References held by someone other than a sequence (a radix-tree span).
  Status retain(const std::vector<int32_t>& block_ids) {
    for (int32_t b : block_ids)
      if (!in_range(b) || ref_[static_cast<size_t>(b)] <= 0)
        return error::InvalidArgument("retain of a block that is not live");
    for (int32_t b : block_ids) change(b, +1);
    return error::Success();
  }
  Status release(const std::vector<int32_t>& block_ids) {
    for (int32_t b : block_ids)
      if (!in_range(b) || ref_[static_cast<size_t>(b)] <= 0)
        return error::InvalidArgument("release of a block that is not live");
    for (int32_t b : block_ids) change(b, -1);
    return error::Success();
  }

  // Row of the block table for the kernels: ids then -1 padding.
  Status fill_block_table_row(int32_t seq, int32_t* row, int32_t max_blocks) const {
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return error::InvalidArgument("unknown sequence");
    const auto& b = it->second.blocks;
    if (static_cast<int32_t>(b.size()) > max_blocks) return error::InvalidArgument("row too short");
    for (int32_t i = 0; i < max_blocks; ++i) row[i] = i < static_cast<int32_t>(b.size()) ? b[static_cast<size_t>(i)] : -1;
    return error::Success();
  }

  // Hands over (and clears) the log of count changes and block copies since the last call.
  void take_pending(std::vector<BlockRefDelta>* deltas, std::vector<BlockCopy>* copies) {
    if (deltas) *deltas = std::move(deltas_);
    if (copies) *copies = std::move(copies_);
    deltas_.clear();
    copies_.clear();
  }
  size_t pending_deltas() const { return deltas_.size(); }
  size_t pending_copies() const { return copies_.size(); }

 private:
  struct Sequence {
    std::vector<int32_t> blocks;
    int32_t length = 0;
  };
  bool in_range(int32_t b) const { return b >= 0 && b < config_.num_blocks; }
  int32_t blocks_for(int32_t tokens) const {
    return (tokens + config_.block_size - 1) / config_.block_size;
  }
  int32_t take_free() {
    const int32_t b = free_.front();
    free_.pop_front();
    change(b, +1);
    return b;
  }
  void change(int32_t b, int32_t delta) {
    int32_t& r = ref_[static_cast<size_t>(b)];
    r += delta;
    deltas_.push_back(BlockRefDelta{b, delta});
    if (r == 0) free_.push_back(b);
  }

  PagedKVConfig config_;
  std::vector<int32_t> ref_;
  std::deque<int32_t> free_;
  std::unordered_map<int32_t, Sequence> seqs_;
  int32_t next_seq_ = 0;
  int64_t cow_events_ = 0;
  std::vector<BlockRefDelta> deltas_;
  std::vector<BlockCopy> copies_;
};

}  // namespace base
#endif  // KUIPER_INCLUDE_BASE_PAGED_KV_H_
