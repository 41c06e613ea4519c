// Host-side bookkeeping of the paged KV pool: 16-token pages handed out from a
// free list, one page-table row per sequence slot.  The pool memory itself
// ([layers] x K/V x [pages, kv_heads, 16, head_dim]) is allocated by the caller;
// this object only decides which page ids a sequence owns and mirrors the table
// into a caller-provided int32 host buffer that is uploaded once per change.
//
// B200 counterpart of the reference's RPUCache geometry (16-token blocked slabs,
// python/rpu_backend/api/cache.py:78-197): one contiguous (16 tokens x local
// heads x head_dim) slab per page.
#include <stdint.h>

#include <memory>
#include <vector>

#include "../common/host_util.h"
#include "../rf_api.h"
#include "handle_registry.h"

namespace rf {

struct KvPool {
  int32_t num_pages = 0, max_seqs = 0, pages_per_seq = 0;
  std::vector<int32_t> free_list;          // LIFO
  std::vector<std::vector<int32_t>> owned; // per sequence slot
};

static HandleRegistry<KvPool>& pools() {
  static HandleRegistry<KvPool> r;
  return r;
}

}  // namespace rf

using namespace rf;

extern "C" int64_t rf_kvpool_create(int32_t num_pages, int32_t max_seqs, int32_t pages_per_seq) {
  if (num_pages <= 0 || max_seqs <= 0 || pages_per_seq <= 0) {
    fail(RF_ERR_BAD_ARG, "kv pool: pages=%d seqs=%d pages_per_seq=%d", num_pages, max_seqs, pages_per_seq);
    return -1;
  }
  auto p = std::make_unique<KvPool>();
  p->num_pages = num_pages; p->max_seqs = max_seqs; p->pages_per_seq = pages_per_seq;
  p->free_list.reserve(num_pages);
  for (int32_t i = num_pages - 1; i >= 0; --i) p->free_list.push_back(i);
  p->owned.resize(max_seqs);
  return pools().insert(std::move(p));
}

extern "C" int rf_kvpool_destroy(int64_t h) {
  return pools().erase(h) ? RF_OK : fail(RF_ERR_BAD_ARG, "unknown kv pool %lld", (long long)h);
}

// Grow sequence `seq` to hold `tokens` tokens; writes the row of the page table
// (pages_per_seq int32, unused entries = 0) into table_row.  RF_ERR_NO_MEMORY if
// the pool or the per-sequence limit is exhausted (nothing is changed then).
extern "C" int rf_kvpool_reserve(int64_t h, int32_t seq, int32_t tokens, int32_t* table_row) {
  auto p = pools().get(h);
  if (!p) return fail(RF_ERR_BAD_ARG, "unknown kv pool %lld", (long long)h);
  RF_REQUIRE(seq >= 0 && seq < p->max_seqs && tokens >= 0, "kv pool: sequence %d / tokens %d", seq, tokens);
  const int32_t need = (tokens + 15) / 16;
  if (need > p->pages_per_seq)
    return fail(RF_ERR_NO_MEMORY, "sequence %d needs %d pages, limit is %d", seq, need, p->pages_per_seq);
  auto& own = p->owned[seq];
  const int32_t extra = need - (int32_t)own.size();
  if (extra > (int32_t)p->free_list.size())
    return fail(RF_ERR_NO_MEMORY, "kv pool exhausted: need %d more pages, %zu free", extra, p->free_list.size());
  for (int32_t i = 0; i < extra; ++i) {
    own.push_back(p->free_list.back());
    p->free_list.pop_back();
  }
  if (table_row) {
    for (int32_t i = 0; i < p->pages_per_seq; ++i) table_row[i] = i < (int32_t)own.size() ? own[i] : 0;
  }
  return RF_OK;
}

extern "C" int rf_kvpool_release(int64_t h, int32_t seq) {
  auto p = pools().get(h);
  if (!p) return fail(RF_ERR_BAD_ARG, "unknown kv pool %lld", (long long)h);
  RF_REQUIRE(seq >= 0 && seq < p->max_seqs, "kv pool: sequence %d", seq);
  auto& own = p->owned[seq];
  for (auto it = own.rbegin(); it != own.rend(); ++it) p->free_list.push_back(*it);
  own.clear();
  return RF_OK;
}

extern "C" int32_t rf_kvpool_free_pages(int64_t h) {
  auto p = pools().get(h);
  return p ? (int32_t)p->free_list.size() : -1;
}
