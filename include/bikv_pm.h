/*
 * bikv_pm.h -- C ABI of the native page directory (part of libbikv.so).
 *
 * The page directory is the coordinator-side table that turns item ids into
 * (shard, page list): the producer of every plan's cache_pages_list.  It is host
 * code only.  Two eviction policies:
 *
 *   BIKV_PM_LRU     the Python coordinator's page managers
 *                   (DistributedStorage/PageManager.py:8-161): per-shard LRU by a
 *                   monotone counter, protected items skipped, a new item goes to
 *                   the shard with most free pages while any shard has more than a
 *                   tenth of its pages free, else to a random shard.
 *   BIKV_PM_TIERED  the Go coordinator's (Go/CacheCoordinator/PageManager.go:101-195,
 *                   306-356,420-526): items are priority 0, user caches priority 2;
 *                   priority 2 is never evicted; a user cache idle for the TTL drops
 *                   to priority 1 at the next clock advance; priority 1 may hold at
 *                   most a quarter of a shard's page count in total, the least
 *                   recently used ones beyond that drop to priority 0; eviction takes
 *                   unprotected entries in (priority, last access) order.
 *
 * Differences from both references, on purpose: time is a logical clock (one tick
 * per operation, or set by bikv_pm_advance_clock) instead of a Python counter /
 * Unix nanoseconds, so runs are reproducible; the free page handed out is always
 * the smallest one (the Python reference's order depends on CPython set
 * internals, the Go one on map iteration order); eviction is O(log n) instead of
 * a sort (Python) or a heap build (Go) over the whole table per eviction; the
 * random shard choice uses the xorshift64* generator documented at
 * bikv_pm_create.  Decisions (hit/miss, shard, which items are evicted, how many
 * pages) are those of the references; page NUMBERS are not, once pages have been
 * recycled.
 *
 * A directory is not thread-safe; calls on one handle must be serialised.
 */
#ifndef BIKV_PM_H_
#define BIKV_PM_H_

#include <stdint.h>

#include "bikv.h"

#ifdef __cplusplus
extern "C" {
#endif

enum bikv_pm_policy { BIKV_PM_LRU = 0, BIKV_PM_TIERED = 1 };

/* Returned by lookups that find nothing (distinct from every bikv_status). */
#define BIKV_PM_MISS (-100)
/* The pool cannot hold the item even with every evictable item gone
 * (the references raise RuntimeError / panic here). */
#define BIKV_PM_FULL (-101)

typedef struct bikv_pm bikv_pm;

/*
 * cache_size_tokens / page_tokens pages per shard (integer division, as both
 * references).  `seed` starts the generator of the random shard choice:
 * x ^= x >> 12; x ^= x << 25; x ^= x >> 27; r = x * 0x2545F4914F6CDD1D;
 * shard = (r >> 33) % n_shards; a zero seed is replaced by 0x9E3779B97F4A7C15.
 * Returns NULL on bad arguments.
 */
bikv_pm* bikv_pm_create(int64_t cache_size_tokens, int32_t page_tokens, int32_t n_shards,
                        int32_t policy, uint64_t seed);
void bikv_pm_destroy(bikv_pm* pm);

/* TIERED only: TTL (in clock units) after which an idle user cache drops to
 * priority 1, and the page quota of priority 1 (default: pages_per_shard / 4). */
int bikv_pm_configure_tiers(bikv_pm* pm, int64_t ttl, int64_t p1_max_pages);

/*
 * MultiPageManager.load_item (PageManager.py:136-154) / LoadItem (PageManager.go:306-356).
 * A known item is only touched (its existing pages come back, *was_cached = 1).
 * Otherwise pages are allocated on the chosen shard, evicting if needed.
 *   weight, is_user   TIERED: weight != 0 gives priority 2; is_user registers the
 *                     item for TTL demotion (the Go code keys this on type "user cache")
 *   out_pages         receives the page numbers (shard-local); capacity `cap`
 *   evicted_out       optional: receives up to evicted_cap evicted item ids
 *   n_evicted         optional: number of items evicted by this call
 * Returns the item's page count, or BIKV_ERR_TOO_LARGE (item larger than a shard;
 * the references raise ValueError / panic), BIKV_PM_FULL, BIKV_ERR_BAD_ARG.
 * If the page list does not fit `cap` the call still completes and returns the
 * count; read the pages with bikv_pm_access_item.
 */
int64_t bikv_pm_load_item(bikv_pm* pm, int64_t item_id, int64_t tokens, int32_t weight,
                          int32_t is_user, int32_t* out_shard, int32_t* out_pages, int64_t cap,
                          int32_t* was_cached, int64_t* evicted_out, int64_t evicted_cap,
                          int64_t* n_evicted);

/* MultiPageManager.access_item (PageManager.py:156-161) / AccessItem
 * (PageManager.go:404-417): touches the item; page count or BIKV_PM_MISS. */
int64_t bikv_pm_access_item(bikv_pm* pm, int64_t item_id, int32_t* out_shard, int32_t* out_pages,
                            int64_t cap);

/* PageManager.set_protected / remove_protected (PageManager.py:91-103): a
 * protected item is skipped by eviction.  BIKV_PM_MISS if the item is unknown. */
int bikv_pm_set_protected(bikv_pm* pm, int64_t item_id);
int bikv_pm_remove_protected(bikv_pm* pm, int64_t item_id);

/* Sets the logical clock (never backwards) and, for TIERED, runs what the Go
 * coordinator's periodic ttlGc does (PageManager.go:488-526): demote idle user
 * caches to priority 1, then enforce the priority-1 quota. */
int bikv_pm_advance_clock(bikv_pm* pm, int64_t now);
/* Sets the logical clock (never backwards) and nothing else.  A caller whose TTL is in
 * wall-clock units calls this with its clock before every batch of decisions, so that the
 * stamps entries receive (clock + 1, + 2, ...) and the `now` of a later
 * bikv_pm_advance_clock share one time base; the Go coordinator stamps entries with
 * time.Now() for the same reason (PageManager.go:488-526 compares against LastAccessed). */
int bikv_pm_set_clock(bikv_pm* pm, int64_t now);

/* Introspection. */
int64_t bikv_pm_free_pages(const bikv_pm* pm, int32_t shard);
int64_t bikv_pm_item_count(const bikv_pm* pm, int32_t shard);
int64_t bikv_pm_evictions(const bikv_pm* pm);
/* Priority of an item (0, 1, 2) or BIKV_PM_MISS. */
int bikv_pm_item_priority(const bikv_pm* pm, int64_t item_id);

/*
 * Plans one worker's share of a prefix-reuse batch natively (the loop of
 * bi-kv_b200/coordinator.py::PrefixCacheCoordinator.plan_batch; decisions as in the
 * coordinator loop of DistributedStorage/CacheCoordinator.py:180-236).  For request
 * i: user[i]'s prefix of prefix_tokens[i] is looked up; a hit yields gather records
 * into worker tensor i at token 0; a miss allocates (evicting LRU items) and yields
 * scatter records at token 0; new_tokens[i] tokens are always stored as a fresh
 * item (ids taken from *next_item_id, which is advanced) and scattered from token
 * prefix_tokens[i].  A user already missed earlier in the same batch is a miss that
 * neither reads nor stores its prefix again.  Every item the batch touches is
 * protected until the batch is planned.  Page ids in the records are GLOBAL for a
 * BIKV_SHARD_BLOCK pool (shard * pages_per_shard + page).
 * Returns 0, or a negative status (capacity, BIKV_PM_FULL, ...).
 */
int bikv_pm_plan_prefix_batch(bikv_pm* pm, const int64_t* users, const int32_t* prefix_tokens,
                              const int32_t* new_tokens, int32_t n_requests, int64_t* next_item_id,
                              bikv_page_rec* gather_out, int64_t gather_cap, int64_t* n_gather,
                              bikv_page_rec* scatter_out, int64_t scatter_cap, int64_t* n_scatter,
                              uint8_t* hit_out);

#ifdef __cplusplus
}
#endif
#endif /* BIKV_PM_H_ */
