/*
 * kpx_kvm.h -- C ABI of the host-side KV-cache manager (lib/libkuiper_b200.so): block pool
 * with reference counts, per-sequence block lists and slot mappings, radix-tree prefix
 * sharing with copy-on-write.  The state lives on the host; every change that the device
 * has to mirror (block reference counts, block copies) is logged and applied by
 * kpx_kvm_flush_device through the kernels of kpx.h.
 *
 * Reference interfaces this stands in for: the position bookkeeping of
 * Model::slice_kv_cache (kuiper/source/model/model.cpp:348-385, one contiguous cache, the
 * position IS the slot) and the PrefixCache round trip of the demo
 * (demo/inference_common.h:757-853,1050-1262: match -> reuse rows in place -> insert ->
 * release).  Paging, sharing by reference and copy-on-write have no reference counterpart.
 */
#ifndef KPX_KVM_H_
#define KPX_KVM_H_
#include <stdint.h>

#include "kpx.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kpx_kvm kpx_kvm;

/* Pool of num_blocks blocks of block_size slots; free list = splitmix64(seed) Fisher-Yates
 * permutation (identity when shuffle == 0).  Prefix cache with the reference's config fields
 * (base::PrefixCacheConfig: max_cached_tokens, min_prefix_length; threshold 0.9, auto
 * eviction and stats on). */
KPX_API kpx_kvm* kpx_kvm_create(int32_t num_blocks, int32_t block_size, uint64_t seed,
                                int32_t shuffle, int64_t max_cached_tokens,
                                int32_t min_prefix_length);
KPX_API void kpx_kvm_destroy(kpx_kvm* m);

/* Sequences.  Functions return a status of kpx.h unless stated otherwise. */
KPX_API int32_t kpx_kvm_add_sequence(kpx_kvm* m); /* -> sequence id >= 0 */
KPX_API int kpx_kvm_append(kpx_kvm* m, int32_t seq, int32_t n, int64_t* slots_out);
KPX_API int kpx_kvm_free_sequence(kpx_kvm* m, int32_t seq);
KPX_API int32_t kpx_kvm_seq_length(const kpx_kvm* m, int32_t seq);     /* -1: unknown */
KPX_API int32_t kpx_kvm_seq_num_blocks(const kpx_kvm* m, int32_t seq); /* -1: unknown */
KPX_API int kpx_kvm_block_table_row(const kpx_kvm* m, int32_t seq, int32_t* row,
                                    int32_t max_blocks);

/* Pool state. */
KPX_API int32_t kpx_kvm_num_free(const kpx_kvm* m);
KPX_API int32_t kpx_kvm_num_shared(const kpx_kvm* m);
KPX_API int64_t kpx_kvm_cow_events(const kpx_kvm* m);
KPX_API int kpx_kvm_ref_counts(const kpx_kvm* m, int32_t* out, int32_t num_blocks);

/* Prefix cache.  match: PrefixCache::match on `tokens`; on a hit the matched blocks are
 * mapped into the (empty) sequence by reference and *matched_out = matched tokens, else 0.
 * insert: the tree takes a reference on the blocks serving the first n tokens of `seq`
 * and records tokens[0..n) -> (0, n).  release: PrefixCache::release. */
KPX_API int kpx_kvm_match_prefix(kpx_kvm* m, int32_t seq, const int32_t* tokens, int32_t n,
                                 int32_t* matched_out);
KPX_API int kpx_kvm_insert_prefix(kpx_kvm* m, int32_t seq, const int32_t* tokens, int32_t n);
KPX_API int kpx_kvm_release_prefix(kpx_kvm* m, const int32_t* tokens, int32_t n);
KPX_API int64_t kpx_kvm_evict(kpx_kvm* m, int64_t target_tokens);
KPX_API int64_t kpx_kvm_cached_tokens(const kpx_kvm* m);
/* out[0..7] = total_requests, cache_hits, cache_misses, total_tokens_processed,
 * tokens_reused, tokens_computed, eviction_count, tokens_evicted */
KPX_API int kpx_kvm_prefix_stats(const kpx_kvm* m, int64_t* out8);

/* Device mirror.  pending: sizes of the logs; take: copy them out and clear them. */
KPX_API int kpx_kvm_pending(const kpx_kvm* m, int32_t* num_deltas, int32_t* num_copies);
KPX_API int kpx_kvm_take_pending(kpx_kvm* m, int32_t* blocks, int32_t* deltas, int32_t cap_deltas,
                                 int32_t* src, int32_t* dst, int32_t cap_copies);
/* Apply the logs on the device: block copies first (copy-on-write, every layer), then the
 * reference-count deltas.  staging_dev: device scratch of at least
 * 8 * (num_deltas + num_copies) bytes (ids then deltas / src then dst).  The host->device
 * copies of the logs are issued on `stream` from pageable memory, which makes them
 * synchronous with respect to the host; the kernels are asynchronous. */
KPX_API int kpx_kvm_flush_device(kpx_kvm* m, int32_t* refcounts_dev, int32_t* error_count_dev,
                                 void* k_pool, void* v_pool, const kpx_kv_layout* layout,
                                 int32_t num_layers, int64_t layer_stride, void* staging_dev,
                                 int64_t staging_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KPX_KVM_H_ */
