// Native page directory: item id -> (shard, pages), LRU or tiered eviction, and
// the prefix-reuse batch planner.  Host code only; contract in include/bikv_pm.h.
#include "bikv_pm.h"

#include <algorithm>
#include <functional>
#include <queue>
#include <set>
#include <tuple>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

struct Entry {
  std::vector<int32_t> pages;
  int64_t last = 0;
  int32_t protect = 0;
  int32_t prio = 0;
  int32_t shard = 0;
};

// (priority, last access, item id): eviction takes the smallest unprotected key.
using OrderKey = std::tuple<int32_t, int64_t, int64_t>;

struct Shard {
  int64_t num_pages = 0;
  std::priority_queue<int32_t, std::vector<int32_t>, std::greater<int32_t>> free_heap;
  std::set<OrderKey> order;  // every entry of this shard with priority 0 or 1
  int64_t items = 0;
};

}  // namespace

struct bikv_pm {
  int32_t policy = BIKV_PM_LRU;
  int32_t page_tokens = 1;
  int64_t pages_per_shard = 0;
  std::vector<Shard> shards;
  std::unordered_map<int64_t, Entry> table;   // item id -> entry (an item lives on one shard)
  std::unordered_set<int64_t> users;          // TIERED: items registered for TTL demotion
  std::set<std::pair<int64_t, int64_t>> p1;   // TIERED: (last access, id) of priority-1 items
  int64_t p1_pages = 0;
  int64_t p1_max_pages = 0;
  int64_t ttl = INT64_MAX;
  int64_t clock = 0;
  int64_t evictions = 0;
  uint64_t rng = 0;

  int64_t tick() { return ++clock; }

  uint32_t random_shard() {
    rng ^= rng >> 12;
    rng ^= rng << 25;
    rng ^= rng >> 27;
    const uint64_t r = rng * 0x2545F4914F6CDD1Dull;
    return (uint32_t)((r >> 33) % (uint64_t)shards.size());
  }

  void order_insert(const Entry& e, int64_t id) {
    if (e.prio == 2) return;
    shards[e.shard].order.emplace(e.prio, e.last, id);
    if (e.prio == 1) p1.emplace(e.last, id);
  }
  void order_erase(const Entry& e, int64_t id) {
    if (e.prio == 2) return;
    shards[e.shard].order.erase(OrderKey(e.prio, e.last, id));
    if (e.prio == 1) p1.erase({e.last, id});
  }

  void touch(Entry& e, int64_t id) {
    order_erase(e, id);
    e.last = tick();
    order_insert(e, id);
  }

  void drop(int64_t id, Entry& e) {  // entry leaves the table; pages go back to the free heap
    order_erase(e, id);
    if (e.prio == 1) p1_pages -= (int64_t)e.pages.size();
    Shard& s = shards[e.shard];
    for (int32_t p : e.pages) s.free_heap.push(p);
    s.items -= 1;
    users.erase(id);
    table.erase(id);
    ++evictions;
  }

  // Evicts from `shard` until `required` pages are free.  Returns false if even
  // evicting every candidate does not suffice (the candidates are gone then, as in
  // both references).
  bool evict(int32_t shard, int64_t required, int64_t* evicted_out, int64_t evicted_cap, int64_t* n_evicted) {
    Shard& s = shards[shard];
    auto it = s.order.begin();
    while ((int64_t)s.free_heap.size() < required && it != s.order.end()) {
      const int64_t id = std::get<2>(*it);
      ++it;  // drop() erases the element `it` pointed at before the increment
      Entry& e = table[id];
      if (e.protect != 0) continue;
      if (n_evicted) {
        if (evicted_out && *n_evicted < evicted_cap) evicted_out[*n_evicted] = id;
        ++*n_evicted;
      }
      drop(id, e);
    }
    return (int64_t)s.free_heap.size() >= required;
  }

  int32_t choose_shard() {
    int64_t most = -1;
    for (const Shard& s : shards) most = std::max<int64_t>(most, (int64_t)s.free_heap.size());
    bool spread;
    if (policy == BIKV_PM_LRU)
      spread = (double)most > (double)pages_per_shard / 10.0;  // PageManager.py:141 (true division)
    else
      spread = most > pages_per_shard / 10;                    // PageManager.go:330 (integer division)
    if (!spread) return (int32_t)random_shard();
    int32_t pick = 0;
    for (int32_t i = 0; i < (int32_t)shards.size(); ++i) {
      if ((int64_t)shards[i].free_heap.size() != most) continue;
      pick = i;
      if (policy == BIKV_PM_LRU) break;  // Python's max() keeps the first, the Go loop the last
    }
    return pick;
  }

  void enforce_p1_quota() {
    while (p1_pages > p1_max_pages && !p1.empty()) {
      const int64_t id = p1.begin()->second;
      Entry& e = table[id];
      order_erase(e, id);
      p1_pages -= (int64_t)e.pages.size();
      e.prio = 0;
      order_insert(e, id);
    }
  }
};

namespace {

int64_t copy_pages(const Entry& e, int32_t* out_shard, int32_t* out_pages, int64_t cap) {
  if (out_shard) *out_shard = e.shard;
  const int64_t n = (int64_t)e.pages.size();
  if (out_pages)
    for (int64_t i = 0; i < std::min(n, cap); ++i) out_pages[i] = e.pages[(size_t)i];
  return n;
}

}  // namespace

extern "C" {

bikv_pm* bikv_pm_create(int64_t cache_size_tokens, int32_t page_tokens, int32_t n_shards, int32_t policy,
                        uint64_t seed) {
  if (cache_size_tokens < 0 || page_tokens <= 0 || n_shards <= 0 || n_shards > 4096) return nullptr;
  if (policy != BIKV_PM_LRU && policy != BIKV_PM_TIERED) return nullptr;
  const int64_t pages = cache_size_tokens / page_tokens;
  if (pages > 0x7fffffffll) return nullptr;
  bikv_pm* pm = new bikv_pm();
  pm->policy = policy;
  pm->page_tokens = page_tokens;
  pm->pages_per_shard = pages;
  pm->p1_max_pages = pages / 4;
  pm->rng = seed ? seed : 0x9E3779B97F4A7C15ull;
  pm->shards.resize((size_t)n_shards);
  for (Shard& s : pm->shards) {
    s.num_pages = pages;
    std::vector<int32_t> all((size_t)pages);
    for (int64_t i = 0; i < pages; ++i) all[(size_t)i] = (int32_t)i;
    s.free_heap = std::priority_queue<int32_t, std::vector<int32_t>, std::greater<int32_t>>(
        std::greater<int32_t>(), std::move(all));
  }
  return pm;
}

void bikv_pm_destroy(bikv_pm* pm) { delete pm; }

int bikv_pm_configure_tiers(bikv_pm* pm, int64_t ttl, int64_t p1_max_pages) {
  if (!pm || ttl < 0 || p1_max_pages < 0) return BIKV_ERR_BAD_ARG;
  pm->ttl = ttl;
  pm->p1_max_pages = p1_max_pages;
  return BIKV_OK;
}

int64_t bikv_pm_access_item(bikv_pm* pm, int64_t item_id, int32_t* out_shard, int32_t* out_pages, int64_t cap) {
  if (!pm || cap < 0) return BIKV_ERR_BAD_ARG;
  auto it = pm->table.find(item_id);
  if (it == pm->table.end()) return BIKV_PM_MISS;
  pm->touch(it->second, item_id);
  return copy_pages(it->second, out_shard, out_pages, cap);
}

int64_t bikv_pm_load_item(bikv_pm* pm, int64_t item_id, int64_t tokens, int32_t weight, int32_t is_user,
                          int32_t* out_shard, int32_t* out_pages, int64_t cap, int32_t* was_cached,
                          int64_t* evicted_out, int64_t evicted_cap, int64_t* n_evicted) {
  if (!pm || tokens < 0 || cap < 0 || evicted_cap < 0) return BIKV_ERR_BAD_ARG;
  if (n_evicted) *n_evicted = 0;
  auto found = pm->table.find(item_id);
  if (found != pm->table.end()) {
    if (was_cached) *was_cached = 1;
    pm->touch(found->second, item_id);
    return copy_pages(found->second, out_shard, out_pages, cap);
  }
  if (was_cached) *was_cached = 0;
  const int64_t required = (tokens + pm->page_tokens - 1) / pm->page_tokens;
  if (required > pm->pages_per_shard) return BIKV_ERR_TOO_LARGE;
  const int32_t shard = pm->choose_shard();
  Shard& s = pm->shards[(size_t)shard];
  if ((int64_t)s.free_heap.size() < required &&
      !pm->evict(shard, required, evicted_out, evicted_cap, n_evicted))
    return BIKV_PM_FULL;
  Entry e;
  e.shard = shard;
  e.pages.reserve((size_t)required);
  for (int64_t i = 0; i < required; ++i) {
    e.pages.push_back(s.free_heap.top());
    s.free_heap.pop();
  }
  e.last = pm->tick();
  e.prio = (pm->policy == BIKV_PM_TIERED && weight != 0) ? 2 : 0;
  if (pm->policy == BIKV_PM_TIERED && is_user) pm->users.insert(item_id);
  s.items += 1;
  Entry& slot = pm->table[item_id];
  slot = std::move(e);
  pm->order_insert(slot, item_id);
  if (pm->policy == BIKV_PM_TIERED) pm->enforce_p1_quota();
  return copy_pages(slot, out_shard, out_pages, cap);
}

int bikv_pm_set_protected(bikv_pm* pm, int64_t item_id) {
  if (!pm) return BIKV_ERR_BAD_ARG;
  auto it = pm->table.find(item_id);
  if (it == pm->table.end()) return BIKV_PM_MISS;
  it->second.protect += 1;
  return BIKV_OK;
}

int bikv_pm_remove_protected(bikv_pm* pm, int64_t item_id) {
  if (!pm) return BIKV_ERR_BAD_ARG;
  auto it = pm->table.find(item_id);
  if (it == pm->table.end()) return BIKV_PM_MISS;
  it->second.protect -= 1;
  return BIKV_OK;
}

int bikv_pm_set_clock(bikv_pm* pm, int64_t now) {
  if (!pm) return BIKV_ERR_BAD_ARG;
  if (now > pm->clock) pm->clock = now;
  return BIKV_OK;
}

int bikv_pm_advance_clock(bikv_pm* pm, int64_t now) {
  if (!pm) return BIKV_ERR_BAD_ARG;
  if (now > pm->clock) pm->clock = now;
  if (pm->policy != BIKV_PM_TIERED) return BIKV_OK;
  std::vector<int64_t> demote;
  for (int64_t id : pm->users) {
    auto it = pm->table.find(id);
    if (it == pm->table.end() || it->second.prio != 2) continue;
    if (pm->clock - it->second.last >= pm->ttl) demote.push_back(id);
  }
  std::sort(demote.begin(), demote.end());
  for (int64_t id : demote) {
    Entry& e = pm->table[id];
    e.prio = 1;
    pm->p1_pages += (int64_t)e.pages.size();
    pm->order_insert(e, id);
    pm->users.erase(id);
  }
  pm->enforce_p1_quota();
  return BIKV_OK;
}

int64_t bikv_pm_free_pages(const bikv_pm* pm, int32_t shard) {
  if (!pm || shard < 0 || shard >= (int32_t)pm->shards.size()) return BIKV_ERR_BAD_ARG;
  return (int64_t)pm->shards[(size_t)shard].free_heap.size();
}

int64_t bikv_pm_item_count(const bikv_pm* pm, int32_t shard) {
  if (!pm || shard < 0 || shard >= (int32_t)pm->shards.size()) return BIKV_ERR_BAD_ARG;
  return pm->shards[(size_t)shard].items;
}

int64_t bikv_pm_evictions(const bikv_pm* pm) { return pm ? pm->evictions : (int64_t)BIKV_ERR_BAD_ARG; }

int bikv_pm_item_priority(const bikv_pm* pm, int64_t item_id) {
  if (!pm) return BIKV_ERR_BAD_ARG;
  auto it = pm->table.find(item_id);
  return it == pm->table.end() ? BIKV_PM_MISS : it->second.prio;
}

int bikv_pm_plan_prefix_batch(bikv_pm* pm, const int64_t* users, const int32_t* prefix_tokens,
                              const int32_t* new_tokens, int32_t n_requests, int64_t* next_item_id,
                              bikv_page_rec* gather_out, int64_t gather_cap, int64_t* n_gather,
                              bikv_page_rec* scatter_out, int64_t scatter_cap, int64_t* n_scatter,
                              uint8_t* hit_out) {
  if (!pm || n_requests < 0 || !next_item_id || !n_gather || !n_scatter || gather_cap < 0 || scatter_cap < 0)
    return BIKV_ERR_BAD_ARG;
  *n_gather = *n_scatter = 0;
  if (n_requests == 0) return BIKV_OK;
  if (!users || !prefix_tokens || !new_tokens || !gather_out || !scatter_out || !hit_out) return BIKV_ERR_BAD_ARG;
  const int32_t P = pm->page_tokens;
  std::vector<int64_t> touched;
  touched.reserve((size_t)n_requests * 2);
  std::unordered_set<int64_t> stored_now;
  int rc = BIKV_OK;

  // Appends the records of one item: its pages cover `tokens` tokens starting at
  // token `at` of worker tensor `req` (short last page as in kvcache.py:169-170).
  auto emit = [&](const Entry& e, int32_t tokens, int32_t req, int32_t at, bikv_page_rec* out, int64_t cap,
                  int64_t* n) -> bool {
    const int64_t count = (int64_t)e.pages.size();
    if (*n + count > cap) return false;
    const int32_t rem = tokens % P;
    for (int64_t k = 0; k < count; ++k) {
      bikv_page_rec& r = out[*n + k];
      r.page_id = (int32_t)((int64_t)e.shard * pm->pages_per_shard + e.pages[(size_t)k]);
      r.valid_tokens = (k == count - 1 && rem != 0) ? rem : P;
      r.request = req;
      r.token_offset = at + (int32_t)k * P;
    }
    *n += count;
    return true;
  };

  for (int32_t i = 0; i < n_requests && rc == BIKV_OK; ++i) {
    const int64_t user = users[i];
    const int32_t prefix = prefix_tokens[i], fresh = new_tokens[i];
    if (prefix < 0 || fresh < 0 || (int64_t)pm->pages_per_shard * (int64_t)pm->shards.size() > 0x7fffffffll) {
      rc = BIKV_ERR_BAD_ARG;
      break;
    }
    auto it = pm->table.find(user);
    if (it != pm->table.end()) pm->touch(it->second, user);
    if (stored_now.count(user)) {
      hit_out[i] = 0;
    } else if (it != pm->table.end()) {
      if ((int64_t)it->second.pages.size() != (prefix + P - 1) / P) {
        rc = BIKV_ERR_PLAN;
        break;
      }
      hit_out[i] = 1;
      if (!emit(it->second, prefix, i, 0, gather_out, gather_cap, n_gather)) rc = BIKV_ERR_TOO_LARGE;
    } else {
      hit_out[i] = 0;
      int32_t shard = 0;
      const int64_t got = bikv_pm_load_item(pm, user, prefix, 0, 0, &shard, nullptr, 0, nullptr, nullptr, 0, nullptr);
      if (got < 0) {
        rc = (int)got;
        break;
      }
      stored_now.insert(user);
      if (!emit(pm->table[user], prefix, i, 0, scatter_out, scatter_cap, n_scatter)) rc = BIKV_ERR_TOO_LARGE;
    }
    if (rc != BIKV_OK) break;
    pm->table[user].protect += 1;
    touched.push_back(user);
    const int64_t item = (*next_item_id)++;
    int32_t shard = 0;
    const int64_t got = bikv_pm_load_item(pm, item, fresh, 0, 0, &shard, nullptr, 0, nullptr, nullptr, 0, nullptr);
    if (got < 0) {
      rc = (int)got;
      break;
    }
    pm->table[item].protect += 1;
    touched.push_back(item);
    if (!emit(pm->table[item], fresh, i, prefix, scatter_out, scatter_cap, n_scatter)) rc = BIKV_ERR_TOO_LARGE;
  }
  for (int64_t id : touched) {
    auto it = pm->table.find(id);
    if (it != pm->table.end()) it->second.protect -= 1;
  }
  return rc;
}

}  // extern "C"
