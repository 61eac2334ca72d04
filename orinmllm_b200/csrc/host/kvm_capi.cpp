// C ABI of the host-side KV-cache manager (include/kpx_kvm.h): base::PagedKVManager and
// base::PrefixCache behind one handle, the tree holding block references through the
// manager, plus the device flush of the pending logs.
#include <cuda_runtime_api.h>

#include <memory>
#include <vector>

#include "base/paged_kv.h"
#include "base/prefix_cache.h"
#include "kpx_kvm.h"

#include "kvm_handle.h"

namespace {
int to_code(const base::Status& s) { return s.get_err_code(); }
std::vector<int32_t> vec(const int32_t* p, int32_t n) {
  return (p && n > 0) ? std::vector<int32_t>(p, p + n) : std::vector<int32_t>();
}
}  // namespace

extern "C" kpx_kvm* kpx_kvm_create(int32_t num_blocks, int32_t block_size, uint64_t seed,
                                   int32_t shuffle, int64_t max_cached_tokens,
                                   int32_t min_prefix_length) {
  if (num_blocks <= 0 || block_size <= 0 || max_cached_tokens <= 0) return nullptr;
  auto* m = new kpx_kvm();
  base::PagedKVConfig pc;
  pc.num_blocks = num_blocks;
  pc.block_size = block_size;
  pc.seed = seed;
  pc.shuffle = shuffle != 0;
  m->pool.reset(new base::PagedKVManager(pc));
  base::PrefixCacheConfig cc;
  cc.max_cached_tokens = max_cached_tokens;
  cc.min_prefix_length = min_prefix_length;
  m->cache.reset(new base::PrefixCache(cc));
  base::PagedKVManager* pool = m->pool.get();
  // a span dropped by the tree (evicted, removed, overwritten, cleared) gives its blocks back
  m->cache->set_block_release_hook([pool](const std::vector<int32_t>& blocks) { pool->release(blocks); });
  return m;
}

extern "C" void kpx_kvm_destroy(kpx_kvm* m) { delete m; }

extern "C" int32_t kpx_kvm_add_sequence(kpx_kvm* m) { return m ? m->pool->add_sequence() : -1; }

extern "C" int kpx_kvm_append(kpx_kvm* m, int32_t seq, int32_t n, int64_t* slots_out) {
  if (!m) return KPX_ERR_INVALID_ARGUMENT;
  std::vector<int64_t> slots;
  base::Status st = m->pool->append(seq, n, &slots);
  if (!st) return to_code(st);
  if (slots_out)
    for (size_t i = 0; i < slots.size(); ++i) slots_out[i] = slots[i];
  return KPX_OK;
}

extern "C" int kpx_kvm_free_sequence(kpx_kvm* m, int32_t seq) {
  return m ? to_code(m->pool->free_sequence(seq)) : KPX_ERR_INVALID_ARGUMENT;
}

extern "C" int32_t kpx_kvm_seq_length(const kpx_kvm* m, int32_t seq) {
  return m ? m->pool->length(seq) : -1;
}

extern "C" int32_t kpx_kvm_seq_num_blocks(const kpx_kvm* m, int32_t seq) {
  if (!m) return -1;
  const std::vector<int32_t>* b = m->pool->blocks(seq);
  return b ? static_cast<int32_t>(b->size()) : -1;
}

extern "C" int kpx_kvm_block_table_row(const kpx_kvm* m, int32_t seq, int32_t* row,
                                       int32_t max_blocks) {
  if (!m || !row || max_blocks < 0) return KPX_ERR_INVALID_ARGUMENT;
  return to_code(m->pool->fill_block_table_row(seq, row, max_blocks));
}

extern "C" int32_t kpx_kvm_num_free(const kpx_kvm* m) { return m ? m->pool->num_free() : -1; }
extern "C" int32_t kpx_kvm_num_shared(const kpx_kvm* m) { return m ? m->pool->num_shared() : -1; }
extern "C" int64_t kpx_kvm_cow_events(const kpx_kvm* m) { return m ? m->pool->cow_events() : -1; }

extern "C" int kpx_kvm_ref_counts(const kpx_kvm* m, int32_t* out, int32_t num_blocks) {
  if (!m || !out || num_blocks != m->pool->config().num_blocks) return KPX_ERR_INVALID_ARGUMENT;
  const std::vector<int32_t>& r = m->pool->ref_counts();
  for (int32_t i = 0; i < num_blocks; ++i) out[i] = r[static_cast<size_t>(i)];
  return KPX_OK;
}

extern "C" int kpx_kvm_match_prefix(kpx_kvm* m, int32_t seq, const int32_t* tokens, int32_t n,
                                    int32_t* matched_out) {
  if (!m || n < 0 || (n > 0 && !tokens) || !m->pool->has_sequence(seq)) return KPX_ERR_INVALID_ARGUMENT;
  if (m->pool->length(seq) != 0) return KPX_ERR_INVALID_ARGUMENT;
  if (matched_out) *matched_out = 0;
  base::PrefixMatchResult r = m->cache->match(vec(tokens, n));
  if (!r.cache_hit) return KPX_OK;
  if (r.block_ids.empty()) {
    // a span inserted without blocks cannot be mapped: hand the reference back, report a miss
    m->cache->release(r.matched_prefix);
    return KPX_OK;
  }
  base::Status st = m->pool->map_prefix(seq, r.block_ids, r.matched_tokens);
  if (!st) {
    m->cache->release(r.matched_prefix);
    return to_code(st);
  }
  if (matched_out) *matched_out = r.matched_tokens;
  return KPX_OK;
}

extern "C" int kpx_kvm_insert_prefix(kpx_kvm* m, int32_t seq, const int32_t* tokens, int32_t n) {
  if (!m || n <= 0 || !tokens) return KPX_ERR_INVALID_ARGUMENT;
  if (m->pool->length(seq) < n) return KPX_ERR_INVALID_ARGUMENT;
  std::vector<int32_t> blocks = m->pool->prefix_blocks(seq, n);
  base::Status st = m->pool->retain(blocks);
  if (!st) return to_code(st);
  m->cache->insert(vec(tokens, n), 0, n, blocks);
  return KPX_OK;
}

extern "C" int kpx_kvm_release_prefix(kpx_kvm* m, const int32_t* tokens, int32_t n) {
  if (!m || n < 0) return KPX_ERR_INVALID_ARGUMENT;
  m->cache->release(vec(tokens, n));
  return KPX_OK;
}

extern "C" int64_t kpx_kvm_evict(kpx_kvm* m, int64_t target_tokens) {
  return m ? m->cache->evict(target_tokens) : -1;
}

extern "C" int64_t kpx_kvm_cached_tokens(const kpx_kvm* m) {
  return m ? m->cache->get_cached_tokens() : -1;
}

extern "C" int kpx_kvm_prefix_stats(const kpx_kvm* m, int64_t* out8) {
  if (!m || !out8) return KPX_ERR_INVALID_ARGUMENT;
  const base::PrefixCacheStats& s = m->cache->get_stats();
  out8[0] = s.total_requests.load();
  out8[1] = s.cache_hits.load();
  out8[2] = s.cache_misses.load();
  out8[3] = s.total_tokens_processed.load();
  out8[4] = s.tokens_reused.load();
  out8[5] = s.tokens_computed.load();
  out8[6] = s.eviction_count.load();
  out8[7] = s.tokens_evicted.load();
  return KPX_OK;
}

extern "C" int kpx_kvm_pending(const kpx_kvm* m, int32_t* num_deltas, int32_t* num_copies) {
  if (!m) return KPX_ERR_INVALID_ARGUMENT;
  if (num_deltas) *num_deltas = static_cast<int32_t>(m->pool->pending_deltas());
  if (num_copies) *num_copies = static_cast<int32_t>(m->pool->pending_copies());
  return KPX_OK;
}

extern "C" int kpx_kvm_take_pending(kpx_kvm* m, int32_t* blocks, int32_t* deltas, int32_t cap_deltas,
                                    int32_t* src, int32_t* dst, int32_t cap_copies) {
  if (!m) return KPX_ERR_INVALID_ARGUMENT;
  if (static_cast<size_t>(cap_deltas) < m->pool->pending_deltas() ||
      static_cast<size_t>(cap_copies) < m->pool->pending_copies())
    return KPX_ERR_WORKSPACE_TOO_SMALL;
  std::vector<base::BlockRefDelta> d;
  std::vector<base::BlockCopy> c;
  m->pool->take_pending(&d, &c);
  for (size_t i = 0; i < d.size(); ++i) {
    blocks[i] = d[i].block;
    deltas[i] = d[i].delta;
  }
  for (size_t i = 0; i < c.size(); ++i) {
    src[i] = c[i].src;
    dst[i] = c[i].dst;
  }
  return KPX_OK;
}

extern "C" int kpx_kvm_flush_device(kpx_kvm* m, int32_t* refcounts_dev, int32_t* error_count_dev,
                                    void* k_pool, void* v_pool, const kpx_kv_layout* layout,
                                    int32_t num_layers, int64_t layer_stride, void* staging_dev,
                                    int64_t staging_bytes, void* stream) {
  if (!m || !refcounts_dev || !staging_dev) return KPX_ERR_INVALID_ARGUMENT;
  const size_t nd = m->pool->pending_deltas(), nc = m->pool->pending_copies();
  if (static_cast<int64_t>(8 * (nd + nc)) > staging_bytes) return KPX_ERR_WORKSPACE_TOO_SMALL;
  if (nc > 0 && (!k_pool || !v_pool || !layout)) return KPX_ERR_INVALID_ARGUMENT;
  std::vector<base::BlockRefDelta> d;
  std::vector<base::BlockCopy> c;
  m->pool->take_pending(&d, &c);
  // The log is ordered; a block may gain and lose references in it.  The kernel applies
  // deltas concurrently and refuses a decrement that would go below zero, so fold the log
  // into one net delta per block first (host order already guarantees the net result).
  std::vector<int32_t> ids, net;
  {
    std::vector<int32_t> acc(static_cast<size_t>(m->pool->config().num_blocks), 0);
    std::vector<int32_t> touched;
    for (const auto& e : d) {
      if (acc[static_cast<size_t>(e.block)] == 0) touched.push_back(e.block);
      acc[static_cast<size_t>(e.block)] += e.delta;
    }
    std::vector<char> seen(acc.size(), 0);
    for (int32_t b : touched) {
      if (seen[static_cast<size_t>(b)]) continue;
      seen[static_cast<size_t>(b)] = 1;
      if (acc[static_cast<size_t>(b)] != 0) {
        ids.push_back(b);
        net.push_back(acc[static_cast<size_t>(b)]);
      }
    }
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t* stage = static_cast<int32_t*>(staging_dev);
  if (!c.empty()) {
    std::vector<int32_t> sd(2 * c.size());
    for (size_t i = 0; i < c.size(); ++i) {
      sd[i] = c[i].src;
      sd[c.size() + i] = c[i].dst;
    }
    if (cudaMemcpyAsync(stage, sd.data(), sd.size() * 4, cudaMemcpyHostToDevice, s) != cudaSuccess)
      return KPX_ERR_CUDA;
    int rc = kpx_cow_copy_blocks(k_pool, v_pool, layout, num_layers, layer_stride, stage,
                                 stage + c.size(), static_cast<int32_t>(c.size()), stream);
    if (rc != KPX_OK) return rc;
    stage += 2 * c.size();
  }
  if (!ids.empty()) {
    std::vector<int32_t> sd(ids);
    sd.insert(sd.end(), net.begin(), net.end());
    if (cudaMemcpyAsync(stage, sd.data(), sd.size() * 4, cudaMemcpyHostToDevice, s) != cudaSuccess)
      return KPX_ERR_CUDA;
    int rc = kpx_refcount_update(refcounts_dev, m->pool->config().num_blocks, stage,
                                 stage + ids.size(), static_cast<int32_t>(ids.size()),
                                 error_count_dev, stream);
    if (rc != KPX_OK) return rc;
  }
  return KPX_OK;
}
