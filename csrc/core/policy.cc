// dSpark verification-length policy (host runtime).
//
// Chooses how many draft rows to verify per round from an online cost/benefit model:
//   benefit(w) = expected emitted tokens = 1 + sum_{j=1..w} prod_{i<=j} a_i      (a_i = calibrated acceptance at depth i)
//   cost(w)    = t_fixed + t_row * (1 + w) + t_draft(w)                          (fitted from device-timed rounds)
// and picks argmax benefit/cost.  Acceptance per depth is an exponentially weighted frequency, optionally conditioned
// on the drafter's confidence through a Platt-style logistic calibration.  Until enough rounds are observed the
// policy verifies everything (warm-up: 12 rounds).  Times come from CUDA events, never host clocks.
// A policy that has settled on plain decoding (width 0) observes nothing any more, so it would never notice that the
// text became predictable again: every `probe_every`-th such decision (64 by default) is answered with a short probe
// of two drafts, whose outcome feeds the acceptance estimate like any other round.
// Rounds shared by several requests are chosen jointly (`ds41_policy_choose_joint`): one target pass verifies all
// blocks, so the round costs  A + B * (rows of all requests)  (fitted from whole-round device times with exponential
// forgetting), every request commits one token whatever is verified, and a draft row adds the probability that the
// whole chain up to it is accepted (per-position probabilities from the drafter's confidence, calibrated online on
// every reached position, blended with the per-depth frequency).  Rows are added in order of decreasing gain while a
// row's gain per microsecond beats the round's average tokens per microsecond, which maximises expected committed tokens
// per predicted round time; a confident request gets a long block, an unsure one may get none.
// Behavioural counterpart of rust/crates/ds41rt-core/src/dspark_policy.rs:449-874 and
// docs/dspark-bandwidth-policy.md:31-140 of the reference (whose cost model is bandwidth balance over RDMA workers;
// here the cost terms are the NVLink-box step times).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

namespace {

struct Policy {
  int max_width;
  int warmup_rounds;
  int rounds = 0;
  std::vector<double> tried, accepted;   // per depth (1-based index - 1), exponentially decayed
  // least squares of round time against rows: t = t_fixed + t_row * rows
  double n = 0, sx = 0, sy = 0, sxx = 0, sxy = 0;
  double draft_us_per_row = 0, draft_n = 0;
  double decay = 0.98;
  // Platt calibration of confidence -> acceptance at depth 1: sigmoid(a*c + b), fitted by SGD
  double pa = 4.0, pb = -2.0;
  uint64_t hist[16] = {0};
  int probe_every = 64, idle = 0;
  uint64_t probes = 0;
  // shared rounds: whole-round time against total rows (exponentially forgotten sums), calibration over all positions
  double jn = 0, jsx = 0, jsy = 0, jsxx = 0, jsxy = 0, jdecay = 0.995;
  double qa = 4.0, qb = -2.0;
  uint64_t joint_rounds = 0, joint_rows_offered = 0, joint_rows_taken = 0;
};

double sigmoid(double x) { return 1.0 / (1.0 + std::exp(-x)); }

}  // namespace

extern "C" {

void* ds41_policy_new(int max_width, int warmup_rounds) {
  Policy* p = new Policy();
  p->max_width = std::max(1, std::min(max_width, 15));
  p->warmup_rounds = warmup_rounds;
  p->tried.assign(p->max_width, 0.0);
  p->accepted.assign(p->max_width, 0.0);
  return p;
}
void ds41_policy_free(void* p) { delete static_cast<Policy*>(p); }

// One verified round: `width` drafts were verified, `n_accepted` of them accepted; device times in microseconds.
void ds41_policy_observe(void* h, int width, int n_accepted, double verify_us, double draft_us, double confidence) {
  Policy* p = static_cast<Policy*>(h);
  width = std::max(0, std::min(width, p->max_width));
  n_accepted = std::max(0, std::min(n_accepted, width));
  for (int d = 0; d < p->max_width; ++d) { p->tried[d] *= p->decay; p->accepted[d] *= p->decay; }
  for (int d = 0; d < width; ++d) {
    if (d <= n_accepted) p->tried[d] += 1.0;          // depth d+1 was reached only if all shallower drafts matched
    if (d < n_accepted) p->accepted[d] += 1.0;
  }
  if (verify_us > 0) {
    const double x = 1.0 + width;
    p->n += 1; p->sx += x; p->sy += verify_us; p->sxx += x * x; p->sxy += x * verify_us;
  }
  if (draft_us > 0 && width > 0) {
    p->draft_us_per_row = (p->draft_us_per_row * p->draft_n + draft_us / width) / (p->draft_n + 1);
    p->draft_n += 1;
  }
  if (confidence >= 0.0 && width > 0) {
    const double y = n_accepted > 0 ? 1.0 : 0.0;
    const double pr = sigmoid(p->pa * confidence + p->pb);
    p->pa += 0.05 * (y - pr) * confidence;
    p->pb += 0.05 * (y - pr);
  }
  ++p->hist[std::min(n_accepted, 15)];
  ++p->rounds;
}

double ds41_policy_acceptance(void* h, int depth) {
  Policy* p = static_cast<Policy*>(h);
  if (depth < 1 || depth > p->max_width) return 0.0;
  const double t = p->tried[depth - 1];
  return t < 1e-9 ? 0.5 : p->accepted[depth - 1] / t;
}

// Number of drafts to verify next round (0..max_width).  `confidence` < 0 means "unknown".
int ds41_policy_choose(void* h, double confidence) {
  Policy* p = static_cast<Policy*>(h);
  if (p->rounds < p->warmup_rounds) return p->max_width;
  double t_fixed = 0.0, t_row = 1.0;
  const double den = p->n * p->sxx - p->sx * p->sx;
  if (p->n >= 2 && std::fabs(den) > 1e-9) {
    t_row = std::max(0.0, (p->n * p->sxy - p->sx * p->sy) / den);
    t_fixed = std::max(0.0, (p->sy - t_row * p->sx) / p->n);
  } else if (p->n >= 1) {
    t_fixed = p->sy / p->n;      // one width seen so far: treat the pass as flat in rows
    t_row = 0.0;
  }
  int best_w = 0;
  double best = -1.0, benefit = 1.0, chain = 1.0;
  for (int w = 0; w <= p->max_width; ++w) {
    if (w > 0) {
      double a = ds41_policy_acceptance(h, w);
      if (w == 1 && confidence >= 0.0) a = 0.5 * a + 0.5 * sigmoid(p->pa * confidence + p->pb);
      chain *= a;
      benefit += chain;
    }
    const double cost = t_fixed + t_row * (1.0 + w) + p->draft_us_per_row * w + 1e-9;
    const double score = benefit / cost;
    if (score > best * (1.0 + 1e-9)) { best = score; best_w = w; }
  }
  if (best_w > 0) {
    p->idle = 0;
  } else if (p->probe_every > 0 && ++p->idle >= p->probe_every) {
    p->idle = 0;
    ++p->probes;
    return std::min(2, p->max_width);
  }
  return best_w;
}

// One shared round as a whole: rows of all requests in the target pass, device time of the round in microseconds.
void ds41_policy_observe_round(void* h, int total_rows, int n_requests, double round_us) {
  Policy* p = static_cast<Policy*>(h);
  if (total_rows <= 0 || n_requests <= 0 || !(round_us > 0)) return;
  const double x = total_rows, d = p->jdecay;
  p->jn = p->jn * d + 1; p->jsx = p->jsx * d + x; p->jsy = p->jsy * d + round_us;
  p->jsxx = p->jsxx * d + x * x; p->jsxy = p->jsxy * d + x * round_us;
  ++p->joint_rounds;
}

// Calibrate the confidence head on every position the verification reached: positions 0..n_accepted-1 were accepted,
// position n_accepted (when verified) was rejected, deeper ones say nothing.
void ds41_policy_observe_positions(void* h, const float* conf, int width, int n_accepted) {
  Policy* p = static_cast<Policy*>(h);
  width = std::max(0, std::min(width, p->max_width));
  n_accepted = std::max(0, std::min(n_accepted, width));
  for (int d = 0; d < width && d <= n_accepted; ++d) {
    const double c = conf[d];
    if (!(c >= 0.0)) continue;
    const double y = d < n_accepted ? 1.0 : 0.0;
    const double pr = sigmoid(p->qa * c + p->qb);
    p->qa += 0.05 * (y - pr) * c;
    p->qb += 0.05 * (y - pr);
  }
}

// Verification lengths of all requests of one shared round.  conf[offsets[r] .. offsets[r+1]) are the drafter's
// confidences of request r's proposed tokens in order (values < 0: unknown).  Writes widths[r] in
// [0, min(offered, max_width)] and returns their sum.
int ds41_policy_choose_joint(void* h, const float* conf, const int* offsets, int n_req, int* widths) {
  Policy* p = static_cast<Policy*>(h);
  int total = 0, offered = 0;
  for (int r = 0; r < n_req; ++r) offered += std::min(offsets[r + 1] - offsets[r], p->max_width);
  p->joint_rows_offered += static_cast<uint64_t>(offered);
  if (p->rounds < p->warmup_rounds) {
    for (int r = 0; r < n_req; ++r) total += widths[r] = std::min(offsets[r + 1] - offsets[r], p->max_width);
    p->joint_rows_taken += static_cast<uint64_t>(total);
    return total;
  }
  // round cost A + B * rows: the whole-round fit when it has seen two row counts, else the per-request fit scaled up
  double A = 0.0, B = 1.0;
  const double jden = p->jn * p->jsxx - p->jsx * p->jsx;
  if (p->jn >= 2 && std::fabs(jden) > 1e-6 * p->jsxx) {
    B = std::max(0.0, (p->jn * p->jsxy - p->jsx * p->jsy) / jden);
    A = std::max(0.0, (p->jsy - B * p->jsx) / p->jn);
  } else if (p->jn >= 1) {
    A = p->jsy / p->jn;
    B = 0.0;
  } else {
    const double den = p->n * p->sxx - p->sx * p->sx;
    double t_fixed = 0.0, t_row = 1.0;
    if (p->n >= 2 && std::fabs(den) > 1e-9) {
      t_row = std::max(0.0, (p->n * p->sxy - p->sx * p->sy) / den);
      t_fixed = std::max(0.0, (p->sy - t_row * p->sx) / p->n);
    } else if (p->n >= 1) {
      t_fixed = p->sy / p->n;
      t_row = 0.0;
    }
    A = t_fixed * n_req;
    B = t_row;
  }
  std::vector<double> chain(n_req, 1.0);
  std::vector<int> w(n_req, 0);
  auto next_gain = [&](int r) -> double {                     // probability that request r's next draft is committed
    const int d = w[r];
    if (d >= std::min(offsets[r + 1] - offsets[r], p->max_width)) return -1.0;
    double a = ds41_policy_acceptance(h, d + 1);
    const double c = conf[offsets[r] + d];
    if (c >= 0.0) a = 0.5 * a + 0.5 * sigmoid(p->qa * c + p->qb);
    return chain[r] * a;
  };
  double tokens = n_req, cost = A + B * n_req + 1e-9;
  for (;;) {
    int best_r = -1;
    double best = 0.0;
    for (int r = 0; r < n_req; ++r) {
      const double g = next_gain(r);
      if (g > best) { best = g; best_r = r; }
    }
    if (best_r < 0 || !(best * cost > tokens * B)) break;       // gain per added cost no longer beats the average
    chain[best_r] = best;
    ++w[best_r];
    tokens += best;
    cost += B;
  }
  for (int r = 0; r < n_req; ++r) total += widths[r] = w[r];
  p->joint_rows_taken += static_cast<uint64_t>(total);
  return total;
}

// out[6]: whole-round fit A, B (microseconds), its sample weight, calibration a, b over all positions, shared rounds;
// counts[2]: draft rows offered to / taken by joint choices.
void ds41_policy_joint_stats(void* h, double* out, uint64_t* counts) {
  Policy* p = static_cast<Policy*>(h);
  const double jden = p->jn * p->jsxx - p->jsx * p->jsx;
  double A = p->jn > 0 ? p->jsy / p->jn : 0.0, B = 0.0;
  if (p->jn >= 2 && std::fabs(jden) > 1e-6 * p->jsxx) {
    B = (p->jn * p->jsxy - p->jsx * p->jsy) / jden;
    A = (p->jsy - B * p->jsx) / p->jn;
  }
  out[0] = A; out[1] = B; out[2] = p->jn; out[3] = p->qa; out[4] = p->qb; out[5] = static_cast<double>(p->joint_rounds);
  counts[0] = p->joint_rows_offered; counts[1] = p->joint_rows_taken;
}

// Probe cadence while the policy chooses plain decoding (0 = never probe); returns the number of probes so far.
uint64_t ds41_policy_probe(void* h, int every) {
  Policy* p = static_cast<Policy*>(h);
  if (every >= 0) p->probe_every = every;
  return p->probes;
}

void ds41_policy_stats(void* h, double* out /*[8]*/, uint64_t* hist16) {
  Policy* p = static_cast<Policy*>(h);
  const double den = p->n * p->sxx - p->sx * p->sx;
  double t_row = 0, t_fixed = p->n > 0 ? p->sy / p->n : 0;
  if (p->n >= 2 && std::fabs(den) > 1e-9) {
    t_row = (p->n * p->sxy - p->sx * p->sy) / den;
    t_fixed = (p->sy - t_row * p->sx) / p->n;
  }
  out[0] = p->rounds; out[1] = t_fixed; out[2] = t_row; out[3] = p->draft_us_per_row;
  out[4] = p->pa; out[5] = p->pb; out[6] = ds41_policy_acceptance(h, 1); out[7] = ds41_policy_acceptance(h, p->max_width);
  for (int i = 0; i < 16; ++i) hist16[i] = p->hist[i];
}

}  // extern "C"
