// Draft-sampling random numbers on the host: the Philox oracle and per-request subsequence reservations.
//
// Every request that samples its drafts owns one Philox subsequence; each draft step reserves a block of counters
// (one counter yields four uniforms, so a vocabulary of V tokens needs ceil(V/4) counters).  Reservations only move
// forward, so a rejected speculative step never reuses numbers, and a forked request takes a fresh subsequence.
// Reference: rust/crates/ds41rt-core/src/dspark_rng.rs (per-request Philox subsequence reservations) and the
// exponential-race draft step in native/cuda/kernels/v41_dspark.cu:241-277.
#include <cstdint>
#include <map>
#include <mutex>

#include "../include/ds41_philox.h"

namespace {
struct Reservations {
  std::mutex mu;
  uint64_t next_subsequence = 1;
  std::map<uint64_t, std::pair<uint64_t, uint64_t>> by_request;   // request -> (subsequence, next offset)
};
}  // namespace

extern "C" {

float ds41_philox_uniform(uint64_t seed, uint64_t subsequence, uint64_t offset, int lane) {
  const ds41::Philox4 r = ds41::philox4x32_10(seed, subsequence, offset);
  return ds41::philox_uniform(r.v[lane & 3]);
}

void* ds41_rng_create() { return new Reservations; }
void ds41_rng_destroy(void* h) { delete static_cast<Reservations*>(h); }

// Reserve `counters` consecutive offsets of the request's subsequence; a request seen for the first time gets the next
// free subsequence.  Returns 0 and fills (subsequence, offset).
int ds41_rng_reserve(void* h, uint64_t request, uint64_t counters, uint64_t* subsequence, uint64_t* offset) {
  auto* r = static_cast<Reservations*>(h);
  if (r == nullptr || subsequence == nullptr || offset == nullptr || counters == 0) return -1;
  std::lock_guard<std::mutex> lk(r->mu);
  auto it = r->by_request.find(request);
  if (it == r->by_request.end()) it = r->by_request.emplace(request, std::make_pair(r->next_subsequence++, 0ull)).first;
  *subsequence = it->second.first;
  *offset = it->second.second;
  it->second.second += counters;
  return 0;
}

// A fork continues with fresh numbers: new subsequence, offset 0.
int ds41_rng_fork(void* h, uint64_t parent, uint64_t child) {
  auto* r = static_cast<Reservations*>(h);
  if (r == nullptr) return -1;
  std::lock_guard<std::mutex> lk(r->mu);
  if (r->by_request.find(parent) == r->by_request.end() || r->by_request.count(child)) return -2;
  r->by_request.emplace(child, std::make_pair(r->next_subsequence++, 0ull));
  return 0;
}

int ds41_rng_release(void* h, uint64_t request) {
  auto* r = static_cast<Reservations*>(h);
  if (r == nullptr) return -1;
  std::lock_guard<std::mutex> lk(r->mu);
  return r->by_request.erase(request) ? 0 : -2;
}

}  // extern "C"
