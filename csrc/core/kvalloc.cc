// Paged KV allocator with generation-checked leases and copy-on-write page sharing (host runtime).
//
// A request holds a lease (slot, generation).  Pages are reference counted so a retained prefix snapshot and the
// requests restored from it share pages; a writer that is about to touch a shared page first takes a private copy
// (the caller performs the device copy for the (src, dst) pair returned).  Revoking a lease bumps the slot's
// generation, so any stale handle is rejected.  Sizing follows the reference's page-group rule
// (rust/crates/ds41rt-daemon/src/v41_native_serve/memory.rs:9-13,137,171-204; leases: v41_requests.rs).
#include <cstdint>
#include <vector>

namespace {

struct Slot {
  uint32_t generation = 1;
  bool active = false;
  std::vector<int32_t> pages;
};

struct Alloc {
  std::vector<int32_t> refs;
  std::vector<int32_t> free_list;
  std::vector<Slot> slots;
  int page_tokens;
};

bool check(const Alloc* a, int slot, uint32_t gen) {
  return slot >= 0 && slot < static_cast<int>(a->slots.size()) && a->slots[slot].active &&
         a->slots[slot].generation == gen;
}

}  // namespace

extern "C" {

void* ds41_kv_new(int n_pages, int n_slots, int page_tokens) {
  if (n_pages <= 0 || n_slots <= 0 || page_tokens <= 0) return nullptr;
  Alloc* a = new Alloc();
  a->refs.assign(n_pages, 0);
  for (int i = n_pages - 1; i >= 0; --i) a->free_list.push_back(i);
  a->slots.resize(n_slots);
  a->page_tokens = page_tokens;
  return a;
}
void ds41_kv_free(void* p) { delete static_cast<Alloc*>(p); }
int ds41_kv_free_pages(const void* p) { return static_cast<int>(static_cast<const Alloc*>(p)->free_list.size()); }

// Admit a request into a free slot: returns the slot (>= 0) and its generation, or -1 when none is free.
int ds41_kv_admit(void* p, uint32_t* generation) {
  Alloc* a = static_cast<Alloc*>(p);
  for (size_t i = 0; i < a->slots.size(); ++i)
    if (!a->slots[i].active) {
      a->slots[i].active = true;
      if (generation) *generation = a->slots[i].generation;
      return static_cast<int>(i);
    }
  return -1;
}

// Admit a request into one particular slot: 0 and its generation, -1 when the slot is taken or out of range.
int ds41_kv_admit_slot(void* p, int slot, uint32_t* generation) {
  Alloc* a = static_cast<Alloc*>(p);
  if (slot < 0 || slot >= static_cast<int>(a->slots.size()) || a->slots[slot].active) return -1;
  a->slots[slot].active = true;
  if (generation) *generation = a->slots[slot].generation;
  return 0;
}
// Generation of an active slot, 0 when the slot is free (generations start at 1).
uint32_t ds41_kv_slot_generation(const void* p, int slot) {
  const Alloc* a = static_cast<const Alloc*>(p);
  if (slot < 0 || slot >= static_cast<int>(a->slots.size()) || !a->slots[slot].active) return 0;
  return a->slots[slot].generation;
}
// Page list of a slot (up to cap entries); returns the number of pages the slot holds.
int ds41_kv_slot_pages(const void* p, int slot, int32_t* out, int cap) {
  const Alloc* a = static_cast<const Alloc*>(p);
  if (slot < 0 || slot >= static_cast<int>(a->slots.size())) return -1;
  const std::vector<int32_t>& pg = a->slots[slot].pages;
  for (int i = 0; i < static_cast<int>(pg.size()) && i < cap; ++i) out[i] = pg[i];
  return static_cast<int>(pg.size());
}

// Ensure pages for positions [0, n_tokens).  Writes newly mapped (index, page) pairs into out (capacity `cap`
// pairs).  Returns the number of new pages, -1 stale lease, -2 pool exhausted (nothing changes), -3 cap too small.
int ds41_kv_ensure(void* p, int slot, uint32_t gen, int n_tokens, int32_t* out, int cap) {
  Alloc* a = static_cast<Alloc*>(p);
  if (!check(a, slot, gen)) return -1;
  Slot& s = a->slots[slot];
  const int need = (n_tokens + a->page_tokens - 1) / a->page_tokens;
  const int have = static_cast<int>(s.pages.size());
  if (need <= have) return 0;
  if (need - have > static_cast<int>(a->free_list.size())) return -2;
  if (need - have > cap) return -3;
  int n = 0;
  for (int i = have; i < need; ++i) {
    const int32_t pg = a->free_list.back();
    a->free_list.pop_back();
    a->refs[pg] = 1;
    s.pages.push_back(pg);
    out[2 * n] = i;
    out[2 * n + 1] = pg;
    ++n;
  }
  return n;
}

// Share the first `n_pages` pages of a retained page list with a slot (prefix restore).
int ds41_kv_share(void* p, int slot, uint32_t gen, const int32_t* pages, int n_pages) {
  Alloc* a = static_cast<Alloc*>(p);
  if (!check(a, slot, gen) || !a->slots[slot].pages.empty()) return -1;
  for (int i = 0; i < n_pages; ++i) {
    if (pages[i] < 0 || pages[i] >= static_cast<int32_t>(a->refs.size()) || a->refs[pages[i]] <= 0) return -2;
  }
  for (int i = 0; i < n_pages; ++i) {
    ++a->refs[pages[i]];
    a->slots[slot].pages.push_back(pages[i]);
  }
  return 0;
}

// Before writing into page index `index`: if it is shared, remap it to a private page.
// Returns 0 (already private), 1 (copied: *src/*dst filled, caller copies the device page), or a negative error.
int ds41_kv_make_private(void* p, int slot, uint32_t gen, int index, int32_t* src, int32_t* dst) {
  Alloc* a = static_cast<Alloc*>(p);
  if (!check(a, slot, gen)) return -1;
  Slot& s = a->slots[slot];
  if (index < 0 || index >= static_cast<int>(s.pages.size())) return -3;
  const int32_t old = s.pages[index];
  if (a->refs[old] == 1) return 0;
  if (a->free_list.empty()) return -2;
  const int32_t fresh = a->free_list.back();
  a->free_list.pop_back();
  a->refs[fresh] = 1;
  --a->refs[old];
  s.pages[index] = fresh;
  if (src) *src = old;
  if (dst) *dst = fresh;
  return 1;
}

// Retain the slot's first n_pages pages for a snapshot (adds a reference each); returns them in out.
int ds41_kv_retain(void* p, int slot, uint32_t gen, int n_pages, int32_t* out) {
  Alloc* a = static_cast<Alloc*>(p);
  if (!check(a, slot, gen) || n_pages > static_cast<int>(a->slots[slot].pages.size())) return -1;
  for (int i = 0; i < n_pages; ++i) {
    out[i] = a->slots[slot].pages[i];
    ++a->refs[out[i]];
  }
  return n_pages;
}

// Drop references held by a snapshot.
void ds41_kv_release_pages(void* p, const int32_t* pages, int n) {
  Alloc* a = static_cast<Alloc*>(p);
  for (int i = 0; i < n; ++i)
    if (pages[i] >= 0 && pages[i] < static_cast<int32_t>(a->refs.size()) && a->refs[pages[i]] > 0 &&
        --a->refs[pages[i]] == 0)
      a->free_list.push_back(pages[i]);
}

// Retire or revoke a lease: its pages lose one reference each and the generation is bumped.
int ds41_kv_retire(void* p, int slot, uint32_t gen) {
  Alloc* a = static_cast<Alloc*>(p);
  if (!check(a, slot, gen)) return -1;
  Slot& s = a->slots[slot];
  ds41_kv_release_pages(p, s.pages.data(), static_cast<int>(s.pages.size()));
  s.pages.clear();
  s.active = false;
  ++s.generation;
  return 0;
}

int ds41_kv_page_count(const void* p, int slot) {
  const Alloc* a = static_cast<const Alloc*>(p);
  return slot >= 0 && slot < static_cast<int>(a->slots.size()) ? static_cast<int>(a->slots[slot].pages.size()) : -1;
}
int ds41_kv_page_ref(const void* p, int page) {
  const Alloc* a = static_cast<const Alloc*>(p);
  return page >= 0 && page < static_cast<int>(a->refs.size()) ? a->refs[page] : -1;
}

// Pool sizing: groups = ceil(ctx / group_tokens) * (slots + 2) + slots + 2 * retained, capped by the byte budget.
long long ds41_kv_plan_groups(long long ctx, int group_tokens, int slots, int retained, long long bytes_per_group,
                              long long budget_bytes) {
  if (group_tokens <= 0 || bytes_per_group <= 0) return -1;
  long long want = (ctx + group_tokens - 1) / group_tokens * (slots + 2) + slots + 2ll * retained;
  const long long fit = budget_bytes / bytes_per_group;
  return want < fit ? want : fit;
}

}  // extern "C"
