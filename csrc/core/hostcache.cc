// Host snapshot cache: a pinned-memory tier behind the device prefix banks (host runtime).
//
// Snapshots evicted from (or written behind) the device banks are kept as lists of fixed-size host pages.  Pages
// are shared exactly: a page whose content key is already resident is reference counted instead of copied.
// Store and restore traffic is rate limited per scheduler tick (byte budgets) so cache traffic cannot starve
// prefill; least-recently-used snapshots are evicted when the slab pool is full.  Copies go through a CopyEngine:
// the real one issues cudaMemcpyAsync (driven from Python), the stub advances a virtual clock with a
// latency + bytes/bandwidth model and can inject failures, which is how the cache is tested without a GPU.
// Behavioural counterpart of rust/crates/ds41rt-hostcache (lib.rs:1-74, copy.rs:37-78, sim.rs:1-50).
#include <algorithm>
#include <cstdint>
#include <map>
#include <unordered_map>
#include <vector>

namespace {

struct Snapshot {
  std::vector<int32_t> pages;
  uint64_t clock;
  uint64_t tokens;
};

struct HostCache {
  int n_pages;
  uint64_t page_bytes;
  std::vector<int32_t> refs;
  std::vector<uint64_t> key_of;
  std::vector<int32_t> free_list;
  std::unordered_map<uint64_t, int32_t> by_key;      // content key -> page
  std::map<int64_t, Snapshot> snaps;
  uint64_t clock = 0;
  // budgets per tick
  uint64_t store_budget, restore_budget, store_used = 0, restore_used = 0;
  // metrics
  uint64_t stored_pages = 0, shared_pages = 0, restored_pages = 0, evictions = 0, hits = 0, misses = 0,
           deferred = 0, failed = 0;
};

struct StubCopy {
  double now_us = 0;
  double latency_us, bytes_per_us;
  uint64_t ops = 0, bytes = 0;
  int64_t fail_at = -1;     // op index that fails (once)
};

void drop_pages(HostCache* c, const std::vector<int32_t>& pages) {
  for (int32_t pg : pages)
    if (--c->refs[pg] == 0) {
      c->by_key.erase(c->key_of[pg]);
      c->free_list.push_back(pg);
    }
}

bool evict_one(HostCache* c, int64_t keep) {
  int64_t victim = -1;
  uint64_t best = ~0ull;
  for (const auto& kv : c->snaps)
    if (kv.first != keep && kv.second.clock < best) { best = kv.second.clock; victim = kv.first; }
  if (victim < 0) return false;
  drop_pages(c, c->snaps[victim].pages);
  c->snaps.erase(victim);
  ++c->evictions;
  return true;
}

}  // namespace

extern "C" {

void* ds41_hostcache_new(int n_pages, uint64_t page_bytes, uint64_t store_budget, uint64_t restore_budget) {
  if (n_pages <= 0 || page_bytes == 0) return nullptr;
  HostCache* c = new HostCache();
  c->n_pages = n_pages;
  c->page_bytes = page_bytes;
  c->refs.assign(n_pages, 0);
  c->key_of.assign(n_pages, 0);
  for (int i = n_pages - 1; i >= 0; --i) c->free_list.push_back(i);
  c->store_budget = store_budget;
  c->restore_budget = restore_budget;
  return c;
}
void ds41_hostcache_free(void* p) { delete static_cast<HostCache*>(p); }
void ds41_hostcache_tick(void* p) {
  HostCache* c = static_cast<HostCache*>(p);
  c->store_used = c->restore_used = 0;
}

// Plan a store of snapshot `id` with per-page content keys.  For each page writes the host page index into
// host_pages[i] and 1 into need_copy[i] when the caller must copy it (0 = already resident, shared).
// Returns n_pages on success, 0 when deferred by the store budget, -1 when the pool cannot hold it even after eviction.
int ds41_hostcache_store(void* p, int64_t id, const uint64_t* keys, int n, uint64_t tokens, int32_t* host_pages,
                         uint8_t* need_copy) {
  HostCache* c = static_cast<HostCache*>(p);
  if (n <= 0 || n > c->n_pages) return -1;
  if (c->snaps.count(id)) { drop_pages(c, c->snaps[id].pages); c->snaps.erase(id); }
  int fresh = 0;
  for (int i = 0; i < n; ++i)
    if (!c->by_key.count(keys[i])) ++fresh;
  if (c->store_used + static_cast<uint64_t>(fresh) * c->page_bytes > c->store_budget) { ++c->deferred; return 0; }
  while (static_cast<int>(c->free_list.size()) < fresh)
    if (!evict_one(c, id)) return -1;
  // eviction may have dropped pages we counted as resident: recount conservatively
  Snapshot s;
  s.clock = ++c->clock;
  s.tokens = tokens;
  for (int i = 0; i < n; ++i) {
    auto it = c->by_key.find(keys[i]);
    if (it != c->by_key.end()) {
      ++c->refs[it->second];
      host_pages[i] = it->second;
      need_copy[i] = 0;
      ++c->shared_pages;
    } else {
      bool room = true;
      while (c->free_list.empty())            // an evicted snapshot may have owned only shared pages
        if (!evict_one(c, id)) { room = false; break; }
      if (!room) { drop_pages(c, s.pages); return -1; }
      const int32_t pg = c->free_list.back();
      c->free_list.pop_back();
      c->refs[pg] = 1;
      c->key_of[pg] = keys[i];
      c->by_key[keys[i]] = pg;
      host_pages[i] = pg;
      need_copy[i] = 1;
      ++c->stored_pages;
      c->store_used += c->page_bytes;
    }
    s.pages.push_back(host_pages[i]);
  }
  c->snaps[id] = std::move(s);
  return n;
}

// A store whose copies failed must be rolled back.
void ds41_hostcache_abort(void* p, int64_t id) {
  HostCache* c = static_cast<HostCache*>(p);
  auto it = c->snaps.find(id);
  if (it == c->snaps.end()) return;
  drop_pages(c, it->second.pages);
  c->snaps.erase(it);
  ++c->failed;
}

// Look up a snapshot for restore.  Returns its page count (pages written to host_pages, capacity `cap`),
// 0 when deferred by the restore budget, -1 when absent.
int ds41_hostcache_restore(void* p, int64_t id, int32_t* host_pages, int cap) {
  HostCache* c = static_cast<HostCache*>(p);
  auto it = c->snaps.find(id);
  if (it == c->snaps.end()) { ++c->misses; return -1; }
  const int n = static_cast<int>(it->second.pages.size());
  if (n > cap) return -1;
  if (c->restore_used + static_cast<uint64_t>(n) * c->page_bytes > c->restore_budget) { ++c->deferred; return 0; }
  c->restore_used += static_cast<uint64_t>(n) * c->page_bytes;
  for (int i = 0; i < n; ++i) host_pages[i] = it->second.pages[i];
  it->second.clock = ++c->clock;
  c->restored_pages += static_cast<uint64_t>(n);
  ++c->hits;
  return n;
}

// The first `n_first` pages of a snapshot, for a prompt that shares only a leading part with it.  Only those pages are
// charged to the restore budget.  Returns n_first, 0 when deferred, -1 when absent or shorter than asked.
int ds41_hostcache_restore_prefix(void* p, int64_t id, int n_first, int32_t* host_pages, int cap) {
  HostCache* c = static_cast<HostCache*>(p);
  auto it = c->snaps.find(id);
  if (it == c->snaps.end()) { ++c->misses; return -1; }
  if (n_first < 0 || n_first > cap || n_first > static_cast<int>(it->second.pages.size())) return -1;
  if (c->restore_used + static_cast<uint64_t>(n_first) * c->page_bytes > c->restore_budget) { ++c->deferred; return 0; }
  c->restore_used += static_cast<uint64_t>(n_first) * c->page_bytes;
  for (int i = 0; i < n_first; ++i) host_pages[i] = it->second.pages[i];
  it->second.clock = ++c->clock;
  c->restored_pages += static_cast<uint64_t>(n_first);
  ++c->hits;
  return n_first;
}

int ds41_hostcache_contains(void* p, int64_t id) { return static_cast<HostCache*>(p)->snaps.count(id) ? 1 : 0; }
int ds41_hostcache_drop(void* p, int64_t id) {
  HostCache* c = static_cast<HostCache*>(p);
  auto it = c->snaps.find(id);
  if (it == c->snaps.end()) return -1;
  drop_pages(c, it->second.pages);
  c->snaps.erase(it);
  return 0;
}

// metrics: [free pages, snapshots, stored, shared, restored, evictions, hits, misses, deferred, failed]
void ds41_hostcache_metrics(void* p, uint64_t* out10) {
  HostCache* c = static_cast<HostCache*>(p);
  out10[0] = c->free_list.size(); out10[1] = c->snaps.size(); out10[2] = c->stored_pages; out10[3] = c->shared_pages;
  out10[4] = c->restored_pages; out10[5] = c->evictions; out10[6] = c->hits; out10[7] = c->misses;
  out10[8] = c->deferred; out10[9] = c->failed;
}

// Invariant check used by the simulator: every page is free xor referenced, reference counts equal the number of
// snapshot slots pointing at the page, and the key map is consistent.  Returns 0 when consistent.
int ds41_hostcache_check(void* p) {
  HostCache* c = static_cast<HostCache*>(p);
  std::vector<int32_t> counted(c->n_pages, 0);
  for (const auto& kv : c->snaps)
    for (int32_t pg : kv.second.pages) {
      if (pg < 0 || pg >= c->n_pages) return 1;
      ++counted[pg];
    }
  std::vector<uint8_t> is_free(c->n_pages, 0);
  for (int32_t pg : c->free_list) {
    if (is_free[pg]) return 2;
    is_free[pg] = 1;
  }
  for (int i = 0; i < c->n_pages; ++i) {
    if (counted[i] != c->refs[i]) return 3;
    if ((c->refs[i] == 0) != (is_free[i] == 1)) return 4;
    if (c->refs[i] > 0) {
      auto it = c->by_key.find(c->key_of[i]);
      if (it == c->by_key.end() || it->second != i) return 5;
    }
  }
  if (c->by_key.size() != static_cast<size_t>(c->n_pages) - c->free_list.size()) return 6;
  return 0;
}

// ---- stub copy engine on a virtual clock
void* ds41_stubcopy_new(double latency_us, double gb_per_s) {
  StubCopy* s = new StubCopy();
  s->latency_us = latency_us;
  s->bytes_per_us = gb_per_s * 1e3;
  return s;
}
void ds41_stubcopy_free(void* p) { delete static_cast<StubCopy*>(p); }
void ds41_stubcopy_fail_at(void* p, int64_t op) { static_cast<StubCopy*>(p)->fail_at = op; }
// returns completion time in virtual microseconds, or a negative value when the copy fails
double ds41_stubcopy_copy(void* p, uint64_t bytes) {
  StubCopy* s = static_cast<StubCopy*>(p);
  const int64_t op = static_cast<int64_t>(s->ops++);
  if (op == s->fail_at) { s->fail_at = -1; return -1.0; }
  s->now_us += s->latency_us + static_cast<double>(bytes) / s->bytes_per_us;
  s->bytes += bytes;
  return s->now_us;
}
double ds41_stubcopy_now(void* p) { return static_cast<StubCopy*>(p)->now_us; }

}  // extern "C"
