// CPU sampler oracle and speculative verification rule (host runtime).
//
// Sampling pipeline per row: allow-mask -> temperature -> min_p -> top_k -> top_p -> categorical draw.
//   inv_T = 1/T; max_scaled = max over allowed (logit * inv_T); min_scaled = max_scaled + ln(min_p) (or -inf);
//   survivors = allowed and scaled >= min_scaled.  Without top_k and with top_p >= 1 the draw is categorical over the
//   survivors in token order.  Otherwise survivors are ranked by (scaled desc, id asc), the top k kept, weights
//   exp(scaled - max) normalised by their sum, the nucleus is the shortest prefix with mass >= top_p, and the draw
//   picks the first rank whose cumulative mass reaches u * nucleus_mass.
//   Greedy when T < 1e-5 or top_k == 1: strict whole-row finiteness, lowest id wins ties.
//   The uniform is SplitMix64 of (seed, position) so a draw depends only on the absolute emitted-token index.
// Behavioural parity: rust/crates/ds41rt-core/src/target_sampling.rs:180-243,421-590 and
// rust/crates/ds41rt-core/src/dspark_verify.rs:18-52 of the reference.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

namespace {

enum Status : int {
  kOk = 0,
  kEmptyCandidates = 1,
  kNonFiniteLogit = 2,
  kInvalidTemperature = 3,
  kMaskWidth = 4,
  kInternal = 5,
  kInvalidParameter = 6,
};

inline bool allowed(const uint32_t* mask, int token) {
  return mask == nullptr || ((mask[token >> 5] >> (token & 31)) & 1u) != 0;
}

}  // namespace

extern "C" {

// Uniform in [0,1) with 24 bits, a pure function of (seed, position).
float ds41_sample_uniform(uint64_t seed, uint64_t position) {
  const uint64_t kDomain = 0x7f4a7c159e3779b9ull;
  const uint64_t kPhi = 0x9e3779b97f4a7c15ull;
  uint64_t x = seed + kDomain + position * kPhi + kPhi;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  x ^= x >> 31;
  return static_cast<float>(static_cast<uint32_t>(x >> 40)) * (1.0f / 16777216.0f);
}

// Returns a Status; *token receives the selected id on kOk.
// top_k <= 0 disables top-k; top_p >= 1 disables the nucleus; min_p <= 0 disables min_p.
int ds41_sample_token(const float* logits, int vocab, const uint32_t* mask, int mask_words, float temperature,
                      int top_k, float top_p, float min_p, float uniform, int* token) {
  if (logits == nullptr || vocab <= 0 || token == nullptr) return kInvalidParameter;
  if (mask != nullptr && mask_words != (vocab + 31) / 32) return kMaskWidth;
  if (!(temperature >= 0.0f) || !std::isfinite(temperature)) return kInvalidTemperature;
  if (!(top_p > 0.0f) || !(min_p >= 0.0f) || min_p > 1.0f) return kInvalidParameter;
  const bool greedy = temperature < 1e-5f || top_k == 1;
  if (greedy) {
    int best = -1;
    float best_v = 0.f;
    for (int i = 0; i < vocab; ++i) {
      if (!std::isfinite(logits[i])) return kNonFiniteLogit;     // strict whole-row finiteness
      if (allowed(mask, i) && (best < 0 || logits[i] > best_v)) { best = i; best_v = logits[i]; }
    }
    if (best < 0) return kEmptyCandidates;
    *token = best;
    return kOk;
  }
  if (!std::isfinite(uniform)) return kInvalidParameter;
  uniform = std::min(std::max(uniform, 0.0f), 0.99999994f);
  const float inv_t = 1.0f / temperature;
  float max_scaled = -std::numeric_limits<float>::infinity();
  int n_allowed = 0;
  for (int i = 0; i < vocab; ++i) {
    if (!allowed(mask, i)) continue;
    if (std::isnan(logits[i]) || logits[i] == std::numeric_limits<float>::infinity()) return kNonFiniteLogit;
    ++n_allowed;
    max_scaled = std::max(max_scaled, logits[i] * inv_t);
  }
  if (n_allowed == 0 || !std::isfinite(max_scaled)) return kEmptyCandidates;
  const float min_scaled = min_p > 0.0f ? max_scaled + std::log(min_p) : -std::numeric_limits<float>::infinity();
  auto survives = [&](int i) { return allowed(mask, i) && logits[i] * inv_t >= min_scaled; };
  const bool filtered = top_k > 0 || top_p < 1.0f;
  if (!filtered) {
    double total = 0.0;
    for (int i = 0; i < vocab; ++i)
      if (survives(i)) total += std::exp(static_cast<double>(logits[i] * inv_t - max_scaled));
    const double target = static_cast<double>(uniform) * total;
    double run = 0.0;
    int last = -1;
    for (int i = 0; i < vocab; ++i) {
      if (!survives(i)) continue;
      run += std::exp(static_cast<double>(logits[i] * inv_t - max_scaled));
      last = i;
      if (run >= target && run > 0.0) { *token = i; return kOk; }
    }
    if (last < 0) return kEmptyCandidates;
    *token = last;
    return kOk;
  }
  std::vector<std::pair<float, int>> ranked;
  ranked.reserve(static_cast<size_t>(n_allowed));
  for (int i = 0; i < vocab; ++i)
    if (survives(i)) ranked.emplace_back(logits[i] * inv_t, i);
  if (ranked.empty()) return kEmptyCandidates;
  auto before = [](const std::pair<float, int>& a, const std::pair<float, int>& b) {
    return a.first > b.first || (a.first == b.first && a.second < b.second);
  };
  size_t keep = ranked.size();
  if (top_k > 0 && static_cast<size_t>(top_k) < keep) {
    keep = static_cast<size_t>(top_k);
    std::partial_sort(ranked.begin(), ranked.begin() + keep, ranked.end(), before);
    ranked.resize(keep);
  } else {
    std::sort(ranked.begin(), ranked.end(), before);
  }
  std::vector<double> w(keep);
  double total = 0.0;
  for (size_t i = 0; i < keep; ++i) {
    w[i] = std::exp(static_cast<double>(ranked[i].first - max_scaled));
    total += w[i];
  }
  size_t nucleus = keep;
  double mass = total;
  if (top_p < 1.0f) {
    double run = 0.0;
    for (size_t i = 0; i < keep; ++i) {
      run += w[i];
      if (run >= static_cast<double>(top_p) * total) { nucleus = i + 1; mass = run; break; }
    }
  }
  const double target = static_cast<double>(uniform) * mass;
  double run = 0.0;
  for (size_t i = 0; i < nucleus; ++i) {
    run += w[i];
    if (run >= target) { *token = ranked[i].second; return kOk; }
  }
  *token = ranked[nucleus - 1].second;
  return kOk;
}

// Speculative verification.  inputs[0] is the anchor, inputs[1..n) the drafts; target_next[i] is the target's choice
// after input row i.  Fills emitted[], returns the number emitted (>= 1) or a negative error.
// *accepted_inputs counts rows whose KV may be committed (anchor + accepted drafts); flags: bit0 EOS, bit1 length.
int ds41_verify_greedy(const uint32_t* inputs, const uint32_t* target_next, int n, uint32_t eos, int remaining,
                       uint32_t vocab, uint32_t* emitted, int* accepted_inputs, int* flags) {
  if (inputs == nullptr || target_next == nullptr || emitted == nullptr || n < 1 || n > 8) return -1;
  if (remaining <= 0 || inputs[0] == eos) return -2;
  for (int i = 0; i < n; ++i)
    if (inputs[i] >= vocab || target_next[i] >= vocab) return -3;
  int acc = 1, count = 0, f = 0;
  for (int i = 0; i < n; ++i) {
    const uint32_t tok = target_next[i];
    const bool matched = i + 1 < n && inputs[i + 1] == tok;
    emitted[count++] = tok;
    if (matched) ++acc;
    const bool is_eos = tok == eos, limit = count == remaining;
    f = (is_eos ? 1 : 0) | (limit ? 2 : 0);
    if (!matched || is_eos || limit) break;
  }
  if (accepted_inputs != nullptr) *accepted_inputs = acc;
  if (flags != nullptr) *flags = f;
  return count;
}

}  // extern "C"
