// radix_trace.cpp -- replays a text script of RadixTree / PrefixCache calls and
// prints every observable result, one line per call.
//
// TEST INFRASTRUCTURE ONLY.  The same source is compiled twice:
//   * against the reference headers (kuiper/include/base/radix_tree.h and
//     prefix_cache.h, taken where they lie in the reference checkout; never
//     copied) -> oracle/_ref/radix_trace_ref, which produced the committed
//     golden outputs under tests/golden/;
//   * against this repository's own headers -> the binary under test.
// Both must print identical text for the same script.
//
// Script grammar (whitespace separated, one call per line, '#' comments):
//   T  insert <start> <len> <n> t0..tn-1      RadixTree::insert
//   T  find   <n> t...                        RadixTree::find_longest_prefix
//   T  contains|remove|addref|release <n> t...
//   T  evict <max_tokens>                     RadixTree::evict_lru
//   T  stats | total | clear
//   P  config <max_cached> <min_prefix> <auto_evict 0|1> <threshold> <stats 0|1>
//   P  match|release|remove <n> t...          PrefixCache::...
//   P  insert <start> <len> <n> t...
//   P  evict <target> | stats | cached | usage | treestats | clear | resetstats
//   tick                                      sleep 2 ms (separates LRU stamps)
// last_access_time (wall clock) and dump() text (unordered_map order) are not
// printed: the reference leaves them unspecified.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "base/radix_tree.h"
#include "base/prefix_cache.h"

static std::vector<int32_t> read_tokens(std::istringstream& in) {
  int n = 0;
  in >> n;
  std::vector<int32_t> t(static_cast<size_t>(n));
  for (int i = 0; i < n; ++i) in >> t[static_cast<size_t>(i)];
  return t;
}

int main(int argc, char** argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: %s <script>\n", argv[0]);
    return 2;
  }
  std::ifstream f(argv[1]);
  if (!f) {
    std::fprintf(stderr, "cannot open %s\n", argv[1]);
    return 2;
  }
  std::unique_ptr<base::RadixTree> tree(new base::RadixTree());
  std::unique_ptr<base::PrefixCache> cache(new base::PrefixCache());
  std::string line;
  long lineno = 0;
  while (std::getline(f, line)) {
    ++lineno;
    if (line.empty() || line[0] == '#') continue;
    std::istringstream in(line);
    std::string who, op;
    in >> who;
    if (who == "tick") {
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
      continue;
    }
    in >> op;
    std::printf("%ld %s %s", lineno, who.c_str(), op.c_str());
    if (who == "T") {
      if (op == "insert") {
        int s, l;
        in >> s >> l;
        auto t = read_tokens(in);
        tree->insert(t, s, l);
        std::printf(" total=%lld", (long long)tree->get_total_cached_tokens());
      } else if (op == "find") {
        auto t = read_tokens(in);
        auto r = tree->find_longest_prefix(t);
        std::printf(" matched=%d edge_offset=%d kv_pos=%d has_kv=%d node=%d", r.matched_length,
                    r.edge_offset, r.kv_cache_pos, r.has_kv_cache() ? 1 : 0,
                    r.matched_node ? 1 : 0);
        if (r.matched_node) {
          const auto& n = *r.matched_node;
          std::printf(" n.prefix_len=%d n.term=%d n.leaf=%d n.edge=%zu n.start=%d n.len=%d n.ref=%d",
                      n.prefix_length, n.is_terminal ? 1 : 0, n.is_leaf() ? 1 : 0,
                      n.edge_tokens.size(), n.kv_info.kv_start_pos, n.kv_info.kv_length,
                      n.kv_info.ref_count);
        }
      } else if (op == "contains") {
        std::printf(" %d", tree->contains(read_tokens(in)) ? 1 : 0);
      } else if (op == "remove") {
        std::printf(" %d", tree->remove(read_tokens(in)) ? 1 : 0);
        std::printf(" total=%lld", (long long)tree->get_total_cached_tokens());
      } else if (op == "addref") {
        tree->add_reference(read_tokens(in));
      } else if (op == "release") {
        tree->release_reference(read_tokens(in));
      } else if (op == "evict") {
        long long m;
        in >> m;
        std::printf(" evicted=%lld", (long long)tree->evict_lru(m));
        std::printf(" total=%lld", (long long)tree->get_total_cached_tokens());
      } else if (op == "stats") {
        auto s = tree->get_stats();
        std::printf(" nodes=%lld terminal=%lld cached=%lld depth=%d", (long long)s.total_nodes,
                    (long long)s.terminal_nodes, (long long)s.total_cached_tokens, s.max_depth);
      } else if (op == "total") {
        std::printf(" %lld", (long long)tree->get_total_cached_tokens());
      } else if (op == "clear") {
        tree->clear();
      } else {
        std::printf(" ?");
      }
    } else if (who == "P") {
      if (op == "config") {
        base::PrefixCacheConfig c;
        int ae, st;
        long long mc;
        in >> mc >> c.min_prefix_length >> ae >> c.eviction_threshold >> st;
        c.max_cached_tokens = mc;
        c.enable_auto_eviction = ae != 0;
        c.enable_stats = st != 0;
        cache.reset(new base::PrefixCache(c));
      } else if (op == "match") {
        auto t = read_tokens(in);
        auto r = cache->match(t);
        std::printf(" hit=%d matched=%d start=%d count=%d ratio=%.9g prefix=%zu", r.cache_hit ? 1 : 0,
                    r.matched_tokens, r.prefill_start_pos, r.prefill_count, (double)r.reuse_ratio,
                    r.matched_prefix.size());
      } else if (op == "insert") {
        int s, l;
        in >> s >> l;
        auto t = read_tokens(in);
        cache->insert(t, s, l);
        std::printf(" cached=%lld", (long long)cache->get_cached_tokens());
      } else if (op == "release") {
        cache->release(read_tokens(in));
      } else if (op == "remove") {
        std::printf(" %d", cache->remove(read_tokens(in)) ? 1 : 0);
      } else if (op == "evict") {
        long long m;
        in >> m;
        std::printf(" evicted=%lld cached=%lld", (long long)cache->evict(m),
                    (long long)cache->get_cached_tokens());
      } else if (op == "stats") {
        const auto& s = cache->get_stats();
        std::printf(" req=%lld hits=%lld miss=%lld tok=%lld reused=%lld computed=%lld evictions=%lld "
                    "evicted=%lld hit_rate=%.9g reuse_rate=%.9g",
                    (long long)s.total_requests.load(), (long long)s.cache_hits.load(),
                    (long long)s.cache_misses.load(), (long long)s.total_tokens_processed.load(),
                    (long long)s.tokens_reused.load(), (long long)s.tokens_computed.load(),
                    (long long)s.eviction_count.load(), (long long)s.tokens_evicted.load(),
                    (double)s.hit_rate(), (double)s.reuse_rate());
      } else if (op == "cached") {
        std::printf(" %lld", (long long)cache->get_cached_tokens());
      } else if (op == "usage") {
        std::printf(" %.9g", (double)cache->get_usage_ratio());
      } else if (op == "treestats") {
        auto s = cache->get_tree_stats();
        std::printf(" nodes=%lld terminal=%lld cached=%lld depth=%d", (long long)s.total_nodes,
                    (long long)s.terminal_nodes, (long long)s.total_cached_tokens, s.max_depth);
      } else if (op == "clear") {
        cache->clear();
      } else if (op == "resetstats") {
        cache->reset_stats();
      } else {
        std::printf(" ?");
      }
    }
    std::printf("\n");
  }
  return 0;
}
