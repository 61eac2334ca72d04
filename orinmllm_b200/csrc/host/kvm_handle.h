// What a kpx_kvm handle points at (shared by the manager and the scheduler C ABIs).
#pragma once
#include <memory>

#include "base/paged_kv.h"
#include "base/prefix_cache.h"

struct kpx_kvm {
  std::unique_ptr<base::PagedKVManager> pool;
  std::unique_ptr<base::PrefixCache> cache;
};
