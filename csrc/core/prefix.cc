// Token-level prefix reuse: a radix tree over token ids with two LRU banks of retained snapshots.
//
// Every retained snapshot records the token sequence it covers (its frontier).  A lookup walks the tree along the
// new prompt and scores each reachable snapshot by the tokens it lets the engine skip:
//     exact ancestor (common == frontier): skipped = common
//     partial match  (common <  frontier): skipped = (common / 2 * 2) - window      (even boundary, replay one window)
// Snapshots live in a Prompt bank or a Turn bank, each with its own capacity and least-recently-used eviction.
// Behavioural parity: rust/crates/ds41rt-core/src/prefix.rs:17-30,234,286-307 of the reference.
#include <cstdint>
#include <map>
#include <memory>
#include <vector>

namespace {

struct Node {
  std::map<uint32_t, std::unique_ptr<Node>> children;
  std::vector<int64_t> snapshots;   // ids whose frontier ends exactly here
  int subtree = 0;                  // snapshots at or below this node
};

struct Snapshot {
  std::vector<uint32_t> tokens;
  int bank;
  uint64_t clock;
  bool live;
};

struct Radix {
  Node root;
  std::vector<Snapshot> snaps;
  uint64_t clock = 0;
  int capacity[2];
  int live[2] = {0, 0};
  int window;
};

void erase_path(Radix* r, int64_t id) {
  const std::vector<uint32_t>& t = r->snaps[id].tokens;
  std::vector<Node*> path{&r->root};
  for (uint32_t tok : t) path.push_back(path.back()->children[tok].get());
  Node* end = path.back();
  for (size_t i = 0; i < end->snapshots.size(); ++i)
    if (end->snapshots[i] == id) { end->snapshots.erase(end->snapshots.begin() + i); break; }
  for (Node* n : path) --n->subtree;
  for (size_t i = path.size() - 1; i > 0; --i)
    if (path[i]->subtree == 0) path[i - 1]->children.erase(t[i - 1]);
    else break;
}

// deepest live snapshot anywhere below `n`; returns id or -1 (any one: they share the common prefix)
int64_t any_below(const Radix* r, const Node* n) {
  if (!n->snapshots.empty()) {
    int64_t best = n->snapshots[0];
    for (int64_t s : n->snapshots)
      if (r->snaps[s].clock > r->snaps[best].clock) best = s;
    return best;
  }
  int64_t best = -1;
  for (const auto& kv : n->children) {
    const int64_t s = any_below(r, kv.second.get());
    if (s >= 0 && (best < 0 || r->snaps[s].clock > r->snaps[best].clock)) best = s;
  }
  return best;
}

}  // namespace

extern "C" {

void* ds41_prefix_new(int prompt_capacity, int turn_capacity, int window) {
  Radix* r = new Radix();
  r->capacity[0] = prompt_capacity;
  r->capacity[1] = turn_capacity;
  r->window = window;
  return r;
}
void ds41_prefix_free(void* p) { delete static_cast<Radix*>(p); }
int ds41_prefix_live(const void* p, int bank) { return static_cast<const Radix*>(p)->live[bank & 1]; }

// Retain a snapshot covering `tokens`.  Returns its id; *evicted receives the id evicted from the bank (or -1).
int64_t ds41_prefix_insert(void* p, const uint32_t* tokens, int n, int bank, int64_t* evicted) {
  Radix* r = static_cast<Radix*>(p);
  bank &= 1;
  if (evicted != nullptr) *evicted = -1;
  if (r->capacity[bank] <= 0) return -1;
  if (r->live[bank] >= r->capacity[bank]) {
    int64_t victim = -1;
    for (size_t i = 0; i < r->snaps.size(); ++i)
      if (r->snaps[i].live && r->snaps[i].bank == bank && (victim < 0 || r->snaps[i].clock < r->snaps[victim].clock))
        victim = static_cast<int64_t>(i);
    if (victim >= 0) {
      erase_path(r, victim);
      r->snaps[victim].live = false;
      --r->live[bank];
      if (evicted != nullptr) *evicted = victim;
    }
  }
  const int64_t id = static_cast<int64_t>(r->snaps.size());
  r->snaps.push_back(Snapshot{std::vector<uint32_t>(tokens, tokens + n), bank, ++r->clock, true});
  Node* node = &r->root;
  ++node->subtree;
  for (int i = 0; i < n; ++i) {
    auto& child = node->children[tokens[i]];
    if (!child) child.reset(new Node());
    node = child.get();
    ++node->subtree;
  }
  node->snapshots.push_back(id);
  ++r->live[bank];
  return id;
}

// Least recently used live snapshot of either bank (-1 when none): the one to drop when the page pool runs short.
int64_t ds41_prefix_oldest(const void* p) {
  const Radix* r = static_cast<const Radix*>(p);
  int64_t victim = -1;
  for (size_t i = 0; i < r->snaps.size(); ++i)
    if (r->snaps[i].live && (victim < 0 || r->snaps[i].clock < r->snaps[victim].clock)) victim = static_cast<int64_t>(i);
  return victim;
}

int ds41_prefix_remove(void* p, int64_t id) {
  Radix* r = static_cast<Radix*>(p);
  if (id < 0 || id >= static_cast<int64_t>(r->snaps.size()) || !r->snaps[id].live) return -1;
  erase_path(r, id);
  r->snaps[id].live = false;
  --r->live[r->snaps[id].bank];
  return 0;
}

// Best reusable snapshot for `tokens`.  Returns its id or -1; *common = matched tokens, *frontier = the snapshot's
// length, *skipped = tokens the engine may skip (reuse score).  Touches the winner's LRU clock.
int64_t ds41_prefix_lookup(void* p, const uint32_t* tokens, int n, int* common, int* frontier, int* skipped) {
  Radix* r = static_cast<Radix*>(p);
  const Node* node = &r->root;
  int64_t best = -1;
  int best_skip = 0, best_common = 0;
  int depth = 0;
  while (true) {
    // exact ancestors ending here
    for (int64_t s : node->snapshots) {
      if (depth > best_skip || (depth == best_skip && best >= 0 && r->snaps[s].clock > r->snaps[best].clock) ||
          (best < 0 && depth >= best_skip)) {
        best = s; best_skip = depth; best_common = depth;
      }
    }
    if (depth == n) break;
    auto it = node->children.find(tokens[depth]);
    if (it == node->children.end()) break;
    node = it->second.get();
    ++depth;
  }
  // partial match: any snapshot strictly below the deepest matched node shares `depth` tokens
  if (depth > 0) {
    int64_t partial = -1;
    for (const auto& kv : node->children) {
      if (depth < n && kv.first == tokens[depth]) continue;
      const int64_t s = any_below(r, kv.second.get());
      if (s >= 0 && (partial < 0 || r->snaps[s].clock > r->snaps[partial].clock)) partial = s;
    }
    if (partial >= 0) {
      const int skip = (depth / 2 * 2) - r->window;
      if (skip > best_skip) { best = partial; best_skip = skip; best_common = depth; }
    }
  }
  if (best < 0 || best_skip <= 0) {
    if (common) *common = 0;
    if (frontier) *frontier = 0;
    if (skipped) *skipped = 0;
    return -1;
  }
  r->snaps[best].clock = ++r->clock;
  if (common) *common = best_common;
  if (frontier) *frontier = static_cast<int>(r->snaps[best].tokens.size());
  if (skipped) *skipped = best_skip;
  return best;
}

}  // extern "C"
