// Engram n-gram hashing and transactional token history (host runtime).
//
// For each of the two Engram layers a token's row ids are hashes of its (2,3,4)-grams over COMPRESSED token ids:
//   rolling = t0*M0; for order 1..3: rolling ^= t[order]*M[order]; for head 0..7:
//   id[(order-1)*8 + head] = rolling % prime[column] + sum of the earlier columns' primes
// where t0 is the current token, t1..t3 the three preceding ones (padding id where history is missing or an
// image/sequence barrier intervenes), the multipliers are model constants and the 24 primes per layer are the
// first primes above 16 000 000 taken consecutively (layer 0 first).  The history commits only accepted tokens:
// prepare() is side-effect free and commit(n) advances by the accepted prefix.
// Behavioural parity: rust/crates/ds41rt-core/src/engram.rs:19-78,141-283 of the reference.
#include <cstdint>
#include <cstring>
#include <mutex>
#include <vector>

namespace {

// Model constants of the official checkpoint (per layer, per n-gram slot).
const uint64_t kMultipliers[2][4] = {
    {76632096046245ull, 4839876093313ull, 35959672319349ull, 73987337458391ull},
    {67716810739261ull, 51510806800915ull, 30921347202721ull, 82619226485591ull},
};

uint64_t g_primes[2][24];
std::once_flag g_once;

bool is_prime(uint64_t n) {
  if (n % 2 == 0) return false;
  for (uint64_t d = 3; d * d <= n; d += 2)
    if (n % d == 0) return false;
  return true;
}

void init_primes() {
  uint64_t c = 16000000ull;
  for (int l = 0; l < 2; ++l)
    for (int i = 0; i < 24; ++i) {
      do { ++c; } while (!is_prime(c));
      g_primes[l][i] = c;
    }
}

struct History {
  uint32_t recent[3];   // recent[0] = most recent committed compressed id
  bool valid[3];
  uint32_t pad;
  uint64_t position;
};

void hash_one(const uint32_t t[4], uint64_t out[2][24]) {
  std::call_once(g_once, init_primes);
  for (int l = 0; l < 2; ++l) {
    uint64_t rolling = static_cast<uint64_t>(t[0]) * kMultipliers[l][0];
    uint64_t offset = 0;
    for (int order = 1; order < 4; ++order) {
      rolling ^= static_cast<uint64_t>(t[order]) * kMultipliers[l][order];
      for (int head = 0; head < 8; ++head) {
        const int col = (order - 1) * 8 + head;
        out[l][col] = rolling % g_primes[l][col] + offset;
        offset += g_primes[l][col];
      }
    }
  }
}

}  // namespace

extern "C" {

void ds41_engram_primes(uint64_t* out48) {
  std::call_once(g_once, init_primes);
  std::memcpy(out48, g_primes, sizeof(g_primes));
}

// tokens[0] = current compressed id, tokens[1..3] = the three preceding ones. out: [2][24].
void ds41_engram_hash(const uint32_t* tokens4, uint64_t* out48) {
  uint64_t tmp[2][24];
  hash_one(tokens4, tmp);
  std::memcpy(out48, tmp, sizeof(tmp));
}

void* ds41_engram_history_new(uint32_t pad_id) {
  History* h = new History();
  for (int i = 0; i < 3; ++i) { h->recent[i] = pad_id; h->valid[i] = false; }
  h->pad = pad_id;
  h->position = 0;
  return h;
}
void ds41_engram_history_free(void* h) { delete static_cast<History*>(h); }
uint64_t ds41_engram_history_position(const void* h) { return static_cast<const History*>(h)->position; }
void* ds41_engram_history_fork(const void* h) { return new History(*static_cast<const History*>(h)); }

// Hash `n` upcoming tokens (compressed ids; negative = image/barrier row) WITHOUT changing the history.
// hashes: [n][2][24]; image rows get zeros and reset the lookback for later rows.
int ds41_engram_prepare(const void* hist, const int32_t* tokens, int n, uint64_t* hashes) {
  if (hist == nullptr || tokens == nullptr || hashes == nullptr || n < 0) return -1;
  History h = *static_cast<const History*>(hist);
  for (int i = 0; i < n; ++i) {
    uint64_t* out = hashes + static_cast<size_t>(i) * 48;
    if (tokens[i] < 0) {
      std::memset(out, 0, 48 * sizeof(uint64_t));
      for (int k = 0; k < 3; ++k) { h.recent[k] = h.pad; h.valid[k] = false; }
      continue;
    }
    uint32_t t[4] = {static_cast<uint32_t>(tokens[i]), h.recent[0], h.recent[1], h.recent[2]};
    uint64_t tmp[2][24];
    hash_one(t, tmp);
    std::memcpy(out, tmp, sizeof(tmp));
    h.recent[2] = h.recent[1]; h.valid[2] = h.valid[1];
    h.recent[1] = h.recent[0]; h.valid[1] = h.valid[0];
    h.recent[0] = t[0]; h.valid[0] = true;
  }
  return 0;
}

// Advance the history by the first `accepted` tokens of a prepared batch (speculative rows beyond leave no trace).
int ds41_engram_commit(void* hist, const int32_t* tokens, int n, int accepted) {
  if (hist == nullptr || tokens == nullptr || accepted < 0 || accepted > n) return -1;
  History* h = static_cast<History*>(hist);
  for (int i = 0; i < accepted; ++i) {
    if (tokens[i] < 0) {
      for (int k = 0; k < 3; ++k) { h->recent[k] = h->pad; h->valid[k] = false; }
    } else {
      h->recent[2] = h->recent[1]; h->valid[2] = h->valid[1];
      h->recent[1] = h->recent[0]; h->valid[1] = h->valid[0];
      h->recent[0] = static_cast<uint32_t>(tokens[i]); h->valid[0] = true;
    }
    ++h->position;
  }
  return 0;
}

}  // extern "C"
