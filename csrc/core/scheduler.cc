// Admission control, lane balancing and round planning (host runtime).
//
//  * Admission: a bounded request queue plus a bounded number of waiters; when both are full the HTTP layer answers
//    429 with Retry-After (reference: rust/crates/ds41rt-api/src/native_v41/admission.rs:15-45).
//  * Lanes: active requests are spread over `lanes` execution lanes so that loads differ by at most one; a retired
//    request triggers a rebalance (reference: rust/crates/ds41rt-daemon/src/v41_native_serve/scheduler.rs:234-241).
//  * Round plan: every member of a lane contributes 1 + draft_len rows, capped by the pass row budget, the request's
//    remaining output budget and its KV room; requests with one remaining token or short history verify the anchor
//    only (docs/ds41-decode-lanes.md:48-49).
#include <algorithm>
#include <cstdint>
#include <mutex>
#include <vector>

namespace {

struct Admission {
  std::mutex mu;
  int queue_cap, waiter_cap;
  int queued = 0, waiting = 0;
  uint64_t accepted = 0, rejected = 0;
};

struct Request {
  int64_t id;
  int lane;
  int remaining;     // output tokens still allowed
  int history;       // tokens already in the sequence
  bool active;
};

struct Lanes {
  int n_lanes;
  std::vector<Request> reqs;
};

}  // namespace

extern "C" {

void* ds41_admission_new(int queue_cap, int waiter_cap) {
  Admission* a = new Admission();
  a->queue_cap = queue_cap;
  a->waiter_cap = waiter_cap;
  return a;
}
void ds41_admission_free(void* p) { delete static_cast<Admission*>(p); }
// 0 = admitted to the queue, 1 = admitted as a waiter (queue full), -1 = rejected (answer 429)
int ds41_admission_reserve(void* p) {
  Admission* a = static_cast<Admission*>(p);
  std::lock_guard<std::mutex> g(a->mu);
  if (a->queued < a->queue_cap) { ++a->queued; ++a->accepted; return 0; }
  if (a->waiting < a->waiter_cap) { ++a->waiting; ++a->accepted; return 1; }
  ++a->rejected;
  return -1;
}
// A queued request left the queue (picked up by the worker or cancelled); a waiter, if any, takes its place.
void ds41_admission_release(void* p) {
  Admission* a = static_cast<Admission*>(p);
  std::lock_guard<std::mutex> g(a->mu);
  if (a->waiting > 0) --a->waiting;
  else if (a->queued > 0) --a->queued;
}
void ds41_admission_stats(void* p, uint64_t* out4) {
  Admission* a = static_cast<Admission*>(p);
  std::lock_guard<std::mutex> g(a->mu);
  out4[0] = static_cast<uint64_t>(a->queued);
  out4[1] = static_cast<uint64_t>(a->waiting);
  out4[2] = a->accepted;
  out4[3] = a->rejected;
}

void* ds41_lanes_new(int n_lanes) {
  Lanes* l = new Lanes();
  l->n_lanes = n_lanes < 1 ? 1 : n_lanes;
  return l;
}
void ds41_lanes_free(void* p) { delete static_cast<Lanes*>(p); }

static void loads(const Lanes* l, std::vector<int>& out) {
  out.assign(l->n_lanes, 0);
  for (const auto& r : l->reqs)
    if (r.active) ++out[r.lane];
}

// Adds a request to the least-loaded lane (lowest index on ties); returns the lane.
int ds41_lanes_add(void* p, int64_t id, int remaining, int history) {
  Lanes* l = static_cast<Lanes*>(p);
  std::vector<int> ld;
  loads(l, ld);
  const int lane = static_cast<int>(std::min_element(ld.begin(), ld.end()) - ld.begin());
  l->reqs.push_back(Request{id, lane, remaining, history, true});
  return lane;
}
int ds41_lanes_update(void* p, int64_t id, int remaining, int history) {
  Lanes* l = static_cast<Lanes*>(p);
  for (auto& r : l->reqs)
    if (r.active && r.id == id) { r.remaining = remaining; r.history = history; return 0; }
  return -1;
}
// Retires a request and rebalances so that lane loads differ by at most one.  Returns the number of moved requests.
int ds41_lanes_retire(void* p, int64_t id) {
  Lanes* l = static_cast<Lanes*>(p);
  bool found = false;
  for (auto& r : l->reqs)
    if (r.active && r.id == id) { r.active = false; found = true; }
  if (!found) return -1;
  l->reqs.erase(std::remove_if(l->reqs.begin(), l->reqs.end(), [](const Request& r) { return !r.active; }),
                l->reqs.end());
  int moved = 0;
  while (true) {
    std::vector<int> ld;
    loads(l, ld);
    const int hi = static_cast<int>(std::max_element(ld.begin(), ld.end()) - ld.begin());
    const int lo = static_cast<int>(std::min_element(ld.begin(), ld.end()) - ld.begin());
    if (ld[hi] - ld[lo] <= 1) break;
    for (auto it = l->reqs.rbegin(); it != l->reqs.rend(); ++it)
      if (it->lane == hi) { it->lane = lo; ++moved; break; }
  }
  return moved;
}
int ds41_lanes_lane_of(void* p, int64_t id) {
  Lanes* l = static_cast<Lanes*>(p);
  for (const auto& r : l->reqs)
    if (r.active && r.id == id) return r.lane;
  return -1;
}
int ds41_lanes_load(void* p, int lane) {
  Lanes* l = static_cast<Lanes*>(p);
  std::vector<int> ld;
  loads(l, ld);
  return lane >= 0 && lane < l->n_lanes ? ld[lane] : -1;
}

// Plans one round of `lane`: ids[i] verifies rows[i] rows (anchor + drafts).  draft_len is the proposal length the
// policy chose; `max_rows` bounds the pass; `min_history` is the history needed before drafts are trusted.
// Returns the number of members written (<= cap).
int ds41_lanes_plan_round(void* p, int lane, int draft_len, int max_rows, int min_history, int64_t* ids, int* rows,
                          int cap) {
  Lanes* l = static_cast<Lanes*>(p);
  int n = 0, used = 0;
  for (const auto& r : l->reqs) {
    if (!r.active || r.lane != lane || r.remaining <= 0 || n >= cap) continue;
    int want = 1 + draft_len;
    if (r.remaining <= 1 || r.history < min_history) want = 1;
    want = std::min(want, r.remaining);          // never verify more rows than tokens may still be emitted
    want = std::min(want, max_rows - used);
    if (want <= 0) break;
    ids[n] = r.id;
    rows[n] = want;
    used += want;
    ++n;
  }
  return n;
}

}  // extern "C"
