// Grammar-mask token sampler on the GPU: one 1024-thread CTA per row.
//
// Same rule as the host oracle (csrc/core/sampler.cc): allow-mask -> temperature -> min_p -> top_k -> top_p ->
// categorical draw with a SplitMix64 (seed, position) uniform; greedy when T < 1e-5 or top_k == 1 (strict whole-row
// finiteness, lowest id wins ties).  Nothing is sorted.  The ranked order (scaled logit descending, id ascending) is
// handled with 8-bit radix selections over an order-preserving integer key:
//   * top-k   : select the k-th largest key by COUNT; ties at that key are admitted lowest id first
//   * top-p   : select by MASS the key at which the cumulative weight reaches top_p * total
//   * the draw: select by MASS the key at which the cumulative weight reaches u * nucleus mass, then the tie index
// Weights exp(scaled - max) are accumulated as 2^-40 fixed point in 64-bit integers, so every sum is independent of
// the order in which threads add and the result is bit-reproducible.  Without top_k / top_p the draw walks the
// survivors in token order (per-thread segments and a block scan), as the oracle does.
// Parity target in the reference: native/cuda/kernels/v41_sampling_gpu.cu:238,523,921,1046,1701 (K1 prepare,
// K2 categorical, K3 top-k pivot, K4 membership / rank order, K5 nucleus) and v41_sampling_gpu.h:52-170.
#include "ds41_api.h"
#include "ds41_launch.cuh"

namespace ds41 {

enum SampleStatus : int {
  kSampleOk = 0,
  kSampleEmpty = 1,
  kSampleNonFinite = 2,
  kSampleBadTemperature = 3,
  kSampleInternal = 5,
  kSampleBadParameter = 6,
};

constexpr int kSampleThreads = 1024;
constexpr double kFx = 1099511627776.0;   // 2^40

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ unsigned long long weight_fx(float scaled, float max_scaled) {
  return static_cast<unsigned long long>(exp(static_cast<double>(scaled - max_scaled)) * kFx + 0.5);
}
__device__ __forceinline__ bool mask_allows(const uint32_t* mask, int i) {
  return mask == nullptr || ((mask[i >> 5] >> (i & 31)) & 1u) != 0;
}
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long position) {
  const unsigned long long kDomain = 0x7f4a7c159e3779b9ull, kPhi = 0x9e3779b97f4a7c15ull;
  unsigned long long x = seed + kDomain + position * kPhi + kPhi;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  x ^= x >> 31;
  return static_cast<float>(static_cast<uint32_t>(x >> 40)) * (1.0f / 16777216.0f);
}

// Walk the row with several independent 16-byte loads in flight per thread (one CTA owns a whole row, so the walk is
// bound by load latency).  Every thread still sees its tokens in ascending order, and every lane of a warp calls
// f(i, value, valid) together, so f may use warp collectives.
template <class F>
__device__ __forceinline__ void for_vocab4(const float* lg, int vocab, F f) {
  const int lane = threadIdx.x & 31, wbase = threadIdx.x - lane, B = blockDim.x;
  constexpr int U = 4;
  if ((reinterpret_cast<uintptr_t>(lg) & 15) == 0) {
    const int n4 = vocab >> 2;
    const float4* lg4 = reinterpret_cast<const float4*>(lg);
    for (int base = wbase; base < n4; base += U * B) {
      float4 v[U];
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int q = base + j * B + lane;
        v[j] = q < n4 ? lg4[q] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < U; ++j) {
        if (base + j * B >= n4) break;
        const int q = base + j * B + lane;
        const bool ok = q < n4;
        f(4 * q, v[j].x, ok);
        f(4 * q + 1, v[j].y, ok);
        f(4 * q + 2, v[j].z, ok);
        f(4 * q + 3, v[j].w, ok);
      }
    }
    if (wbase == 0 && 4 * n4 < vocab) {          // up to three trailing tokens, warp 0
      const int i = 4 * n4 + lane;
      f(i, i < vocab ? lg[i] : 0.f, i < vocab);
    }
    return;
  }
  for (int base = wbase; base < vocab; base += U * B) {
    float v[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int i = base + j * B + lane;
      v[j] = i < vocab ? lg[i] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int i = base + j * B + lane;
      if (base + j * B < vocab) f(i, v[j], i < vocab);
    }
  }
}

constexpr int kSampleListCap = 2048;   // survivors of a top-k cut are kept in shared memory up to this many

struct SampleShared {
  float list_val[kSampleListCap];       // raw logits of the tokens above the top-k cut key (any order)
  int list_id[kSampleListCap];
  int list_n;
  unsigned int cnt[256];
  unsigned long long mass[256];
  unsigned long long scan[kSampleThreads];
  unsigned long long total;
  double remaining;
  unsigned int digit, tie_count;
  int flag, token;
  float fmax;
  int imax;
};

// What a selection walks: the whole row, or (n_list >= 0) the compact list of the tokens above the top-k cut key.
struct RowView {
  const float* lg;
  int vocab;
  const uint32_t* mask;
  const float* list_val;
  const int* list_id;
  int n_list;
};

template <class F>
__device__ __forceinline__ void for_view(const RowView& v, F f) {
  if (v.n_list < 0) {
    for_vocab4(v.lg, v.vocab, [&](int i, float x, bool valid) { f(i, x, valid && mask_allows(v.mask, i)); });
    return;
  }
  const int lane = threadIdx.x & 31, wbase = threadIdx.x - lane;
  for (int base = wbase; base < v.n_list; base += blockDim.x) {
    const int j = base + lane;
    const bool valid = j < v.n_list;
    f(valid ? v.list_id[j] : 0, valid ? v.list_val[j] : 0.f, valid);
  }
}

// The candidate set of a selection: allowed tokens with key > excl, plus `tie_mult` tokens of key `tie_key`
// (the admitted part of a tie group cut by an earlier selection; tie_key <= excl whenever tie_mult > 0).
struct CandSet {
  uint32_t excl;
  uint32_t tie_key;
  unsigned long long tie_mult;
};

// Radix selection, high keys first.  by_mass: find the key at which the running weight reaches `target`; else the key
// at which the running count reaches it.  On return sh.remaining is what the ties at the returned key must still
// supply and sh.tie_count how many candidates carry that key.
__device__ uint32_t radix_select(SampleShared& sh, const RowView& view, float inv_t, float max_scaled, CandSet set,
                                 bool by_mass, double target) {
  uint32_t prefix = 0, prefix_mask = 0;
  if (threadIdx.x == 0) sh.remaining = target;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int d = threadIdx.x; d < 256; d += blockDim.x) {
      sh.cnt[d] = 0;
      sh.mass[d] = 0;
    }
    __syncthreads();
    // lanes of a warp that hit the same digit add once: logits of one row share their top key bytes, so unaggregated
    // shared-memory atomics would serialise on a handful of counters.  Integer sums: the result does not depend on
    // the grouping.
    for_view(view, [&](int i, float v, bool valid) {
      const float s = __fmul_rn(v, inv_t);
      const uint32_t k = order_key(s);
      const bool act = valid && k > set.excl && (k & prefix_mask) == prefix;
      const uint32_t d = (k >> shift) & 255u;
      const unsigned peers = __match_any_sync(0xffffffffu, act ? d : 256u);
      if (act) {
        const int leader = __ffs(peers) - 1;
        const int lane = threadIdx.x & 31;
        unsigned long long wsum = 0;
        if (by_mass) {
          const unsigned long long w = weight_fx(s, max_scaled);           // <= 2^40: two 20/21-bit halves
          const unsigned lo = __reduce_add_sync(peers, static_cast<unsigned>(w & 0xFFFFFu));
          const unsigned hi = __reduce_add_sync(peers, static_cast<unsigned>(w >> 20));
          wsum = (static_cast<unsigned long long>(hi) << 20) + lo;
        }
        if (lane == leader) {
          atomicAdd(&sh.cnt[d], static_cast<unsigned>(__popc(peers)));
          if (by_mass) atomicAdd(&sh.mass[d], wsum);
        }
      }
    });
    if (threadIdx.x == 0 && set.tie_mult > 0 && (set.tie_key & prefix_mask) == prefix) {
      const uint32_t d = (set.tie_key >> shift) & 255u;
      atomicAdd(&sh.cnt[d], static_cast<unsigned int>(set.tie_mult));
      if (by_mass) atomicAdd(&sh.mass[d], set.tie_mult * weight_fx(key_value(set.tie_key), max_scaled));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      double acc = 0.0;
      int pick = -1, lowest = -1;
      for (int d = 255; d >= 0; --d) {
        if (sh.cnt[d] == 0) continue;
        lowest = d;
        const double v = by_mass ? static_cast<double>(sh.mass[d]) : static_cast<double>(sh.cnt[d]);
        if (acc + v >= sh.remaining) { pick = d; break; }
        acc += v;
      }
      if (pick < 0) {           // rounding left the target just above the total: end on the lowest key present
        pick = lowest < 0 ? 0 : lowest;
        acc -= by_mass ? static_cast<double>(sh.mass[pick]) : static_cast<double>(sh.cnt[pick]);
        if (acc < 0.0) acc = 0.0;
      }
      sh.remaining -= acc;
      sh.digit = static_cast<unsigned int>(pick);
      sh.tie_count = sh.cnt[pick];
    }
    __syncthreads();
    prefix |= sh.digit << shift;
    prefix_mask |= 255u << shift;
    __syncthreads();
  }
  return prefix;
}

// Block-wide exclusive scan of one value per thread (Hillis-Steele in shared memory); returns the exclusive prefix and
// leaves the grand total in sh.total.
__device__ unsigned long long block_scan(SampleShared& sh, unsigned long long v) {
  sh.scan[threadIdx.x] = v;
  __syncthreads();
  for (int off = 1; off < kSampleThreads; off <<= 1) {
    const unsigned long long add = threadIdx.x >= off ? sh.scan[threadIdx.x - off] : 0ull;
    __syncthreads();
    sh.scan[threadIdx.x] += add;
    __syncthreads();
  }
  const unsigned long long incl = sh.scan[threadIdx.x];
  if (threadIdx.x == kSampleThreads - 1) sh.total = incl;
  __syncthreads();
  return incl - v;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, long long ld, int vocab, const uint32_t* __restrict__ masks,
                   int mask_words, const ds41_sample_row* __restrict__ rows, int* __restrict__ tokens,
                   int* __restrict__ status) {
  __shared__ SampleShared sh;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const ds41_sample_row p = rows[row];
  const float* lg = logits + 1ll * row * ld;
  const uint32_t* mask = (masks != nullptr && p.mask_row >= 0) ? masks + 1ll * p.mask_row * mask_words : nullptr;
  const int tid = threadIdx.x;
  auto finish = [&](int st, int tok) {
    if (tid == 0) {
      status[row] = st;
      if (st == kSampleOk) tokens[row] = tok;
    }
  };
  if (!(p.temperature >= 0.0f) || isinf(p.temperature)) return finish(kSampleBadTemperature, 0);
  if (!(p.top_p > 0.0f) || !(p.min_p >= 0.0f) || p.min_p > 1.0f) return finish(kSampleBadParameter, 0);
  if (tid == 0) { sh.flag = 0; sh.fmax = -INFINITY; sh.imax = -1; }
  __syncthreads();
  const bool greedy = p.temperature < 1e-5f || p.top_k == 1;
  const float inv_t = greedy ? 1.0f : 1.0f / p.temperature;

  // ---- prepare: finiteness, allowed count, maximum (greedy: arg max with the lowest id on ties)
  float best = -INFINITY;
  int best_i = -1, n_allowed = 0, bad = 0;
  for_vocab4(lg, vocab, [&](int i, float v, bool valid) {
    if (!valid) return;
    const bool ok = mask_allows(mask, i);
    if (greedy) {
      if (!isfinite(v)) bad = 1;
    } else if (ok && (isnan(v) || v == INFINITY)) {
      bad = 1;
    }
    if (!ok) return;
    ++n_allowed;
    const float s = __fmul_rn(v, inv_t);
    if (best_i < 0 || s > best) { best = s; best_i = i; }      // ascending i per thread: first maximum kept
  });
  for (int off = 16; off > 0; off >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
    n_allowed += __shfl_xor_sync(0xffffffffu, n_allowed, off);
    bad |= __shfl_xor_sync(0xffffffffu, bad, off);
    if (oi >= 0 && (best_i < 0 || ob > best || (ob == best && oi < best_i))) { best = ob; best_i = oi; }
  }
  if ((tid & 31) == 0) {
    sh.scan[tid >> 5] = (static_cast<unsigned long long>(__float_as_uint(best)) << 32) | static_cast<uint32_t>(best_i);
    sh.cnt[tid >> 5] = static_cast<unsigned int>(n_allowed);
    if (bad) atomicOr(&sh.flag, 1);
  }
  __syncthreads();
  if (tid == 0) {
    float b = -INFINITY;
    int bi = -1;
    unsigned int n = 0;
    for (int w = 0; w < kSampleThreads / 32; ++w) {
      const float ob = __uint_as_float(static_cast<uint32_t>(sh.scan[w] >> 32));
      const int oi = static_cast<int>(static_cast<uint32_t>(sh.scan[w]));
      n += sh.cnt[w];
      if (oi >= 0 && (bi < 0 || ob > b || (ob == b && oi < bi))) { b = ob; bi = oi; }
    }
    sh.fmax = b;
    sh.imax = bi;
    sh.tie_count = n;
  }
  __syncthreads();
  if (sh.flag) return finish(kSampleNonFinite, 0);
  if (sh.imax < 0 || sh.tie_count == 0) return finish(kSampleEmpty, 0);
  if (greedy) return finish(kSampleOk, sh.imax);
  const float max_scaled = sh.fmax;
  if (!isfinite(max_scaled)) return finish(kSampleEmpty, 0);
  __syncthreads();

  const float u = fminf(fmaxf(uniform01(p.seed, p.position), 0.0f), 0.99999994f);
  const float min_scaled = p.min_p > 0.0f ? max_scaled + logf(p.min_p) : -INFINITY;
  // survivors: key >= key(min_scaled)  <=>  key > excl
  const uint32_t excl0 = p.min_p > 0.0f ? order_key(min_scaled) - 1u : 0u;
  const bool filtered = p.top_k > 0 || p.top_p < 1.0f;

  if (!filtered) {
    // ---- categorical over the survivors in token order
    const int seg = (vocab + kSampleThreads - 1) / kSampleThreads;
    const int i0 = min(vocab, tid * seg), i1 = min(vocab, i0 + seg);
    unsigned long long mine = 0;
    for (int i = i0; i < i1; ++i) {
      if (!mask_allows(mask, i)) continue;
      const float s = __fmul_rn(lg[i], inv_t);
      if (order_key(s) > excl0) mine += weight_fx(s, max_scaled);
    }
    const unsigned long long before = block_scan(sh, mine);
    const double target = static_cast<double>(u) * static_cast<double>(sh.total);
    if (tid == 0) sh.token = -1;
    __syncthreads();
    // the first thread whose inclusive sum reaches the target owns the draw
    if (mine > 0 && static_cast<double>(before + mine) >= target &&
        (static_cast<double>(before) < target || before == 0)) {
      unsigned long long run = before;
      for (int i = i0; i < i1; ++i) {
        if (!mask_allows(mask, i)) continue;
        const float s = __fmul_rn(lg[i], inv_t);
        if (order_key(s) <= excl0) continue;
        run += weight_fx(s, max_scaled);
        if (static_cast<double>(run) >= target && run > 0) { atomicCAS(&sh.token, -1, i); break; }
      }
    }
    __syncthreads();
    if (sh.token < 0) {
      // rounding: nothing reached the target - the last survivor wins
      int last = -1;
      for (int i = i1 - 1; i >= i0; --i) {
        if (mask_allows(mask, i) && order_key(__fmul_rn(lg[i], inv_t)) > excl0) { last = i; break; }
      }
      if (last >= 0) atomicMax(&sh.token, last);
      __syncthreads();
    }
    return finish(sh.token >= 0 ? kSampleOk : kSampleEmpty, sh.token);
  }

  // ---- ranked path
  CandSet set{excl0, 0u, 0ull};
  RowView view{lg, vocab, mask, sh.list_val, sh.list_id, -1};
  // survivor count
  int mine_n = 0;
  for_view(view, [&](int i, float v, bool valid) {
    if (valid && order_key(__fmul_rn(v, inv_t)) > excl0) ++mine_n;
  });
  block_scan(sh, static_cast<unsigned long long>(mine_n));
  const unsigned long long survivors = sh.total;
  __syncthreads();
  if (survivors == 0) return finish(kSampleEmpty, 0);
  uint32_t list_key = 0xFFFFFFFFu;      // keys above this one live in the compact list (when view.n_list >= 0)
  if (p.top_k > 0 && static_cast<unsigned long long>(p.top_k) < survivors) {
    const uint32_t pk = radix_select(sh, view, inv_t, max_scaled, set, false, static_cast<double>(p.top_k));
    const double need = sh.remaining;
    const unsigned long long ties = sh.tie_count;
    __syncthreads();
    set.excl = pk;
    set.tie_key = pk;
    set.tie_mult = static_cast<unsigned long long>(fmin(fmax(need, 1.0), static_cast<double>(ties)));
    if (p.top_k <= kSampleListCap) {
      // fewer than top_k tokens lie above the cut key: gather them once; every later selection walks this list
      // instead of the row (the admitted ties of the cut key stay described by set.tie_key / set.tie_mult)
      if (tid == 0) sh.list_n = 0;
      __syncthreads();
      for_view(view, [&](int i, float v, bool valid) {
        const bool keep = valid && order_key(__fmul_rn(v, inv_t)) > pk;
        const unsigned m = __ballot_sync(0xffffffffu, keep);
        if (m == 0) return;
        const int lane = threadIdx.x & 31;
        int at = 0;
        if (lane == __ffs(m) - 1) at = atomicAdd(&sh.list_n, __popc(m));
        at = __shfl_sync(0xffffffffu, at, __ffs(m) - 1) + __popc(m & ((1u << lane) - 1u));
        if (keep && at < kSampleListCap) {
          sh.list_val[at] = v;
          sh.list_id[at] = i;
        }
      });
      __syncthreads();
      if (sh.list_n <= kSampleListCap) {
        view.n_list = sh.list_n;
        list_key = pk;
      }
    }
  }
  // total weight of the kept set
  unsigned long long mine_w = 0;
  for_view(view, [&](int i, float v, bool valid) {
    if (!valid) return;
    const float s = __fmul_rn(v, inv_t);
    if (order_key(s) > set.excl) mine_w += weight_fx(s, max_scaled);
  });
  block_scan(sh, mine_w);
  unsigned long long total = sh.total + set.tie_mult * (set.tie_mult ? weight_fx(key_value(set.tie_key), max_scaled) : 0ull);
  __syncthreads();
  double mass = static_cast<double>(total);
  if (p.top_p < 1.0f) {
    const double target = static_cast<double>(p.top_p) * mass;
    const uint32_t pp = radix_select(sh, view, inv_t, max_scaled, set, true, target);
    const double need = sh.remaining;
    const unsigned long long ties = sh.tie_count;
    __syncthreads();
    const double w = static_cast<double>(weight_fx(key_value(pp), max_scaled));
    unsigned long long take = w > 0.0 ? static_cast<unsigned long long>(ceil(need / w)) : ties;
    if (take < 1) take = 1;
    if (take > ties) take = ties;
    mass = (target - need) + static_cast<double>(take) * w;
    set.excl = pp;
    set.tie_key = pp;
    set.tie_mult = take;
  }
  // ---- the draw
  const double target = static_cast<double>(u) * mass;
  const uint32_t dk = radix_select(sh, view, inv_t, max_scaled, set, true, target);
  const double need = sh.remaining;
  const unsigned long long ties = sh.tie_count;
  __syncthreads();
  const double w = static_cast<double>(weight_fx(key_value(dk), max_scaled));
  long long tie_index = w > 0.0 ? static_cast<long long>(ceil(need / w)) - 1 : 0;
  if (tie_index < 0) tie_index = 0;
  if (tie_index > static_cast<long long>(ties) - 1) tie_index = static_cast<long long>(ties) - 1;
  // the tie_index-th allowed token with key == dk in id order
  if (view.n_list >= 0 && dk > list_key) {
    // all tokens of that key are in the list: the one with exactly tie_index smaller ids among them
    if (tid == 0) sh.token = -1;
    __syncthreads();
    for (int j = tid; j < view.n_list; j += blockDim.x) {
      if (order_key(__fmul_rn(sh.list_val[j], inv_t)) != dk) continue;
      long long rank = 0;
      for (int q = 0; q < view.n_list; ++q)
        if (sh.list_id[q] < sh.list_id[j] && order_key(__fmul_rn(sh.list_val[q], inv_t)) == dk) ++rank;
      if (rank == tie_index) sh.token = sh.list_id[j];
    }
    __syncthreads();
    return finish(sh.token >= 0 ? kSampleOk : kSampleInternal, sh.token);
  }
  const int seg = (vocab + kSampleThreads - 1) / kSampleThreads;
  const int i0 = min(vocab, tid * seg), i1 = min(vocab, i0 + seg);
  unsigned long long eq = 0;
  for (int i = i0; i < i1; ++i)
    if (mask_allows(mask, i) && order_key(__fmul_rn(lg[i], inv_t)) == dk) ++eq;
  const unsigned long long before = block_scan(sh, eq);
  if (tid == 0) sh.token = -1;
  __syncthreads();
  if (eq > 0 && static_cast<long long>(before) <= tie_index && tie_index < static_cast<long long>(before + eq)) {
    long long seen = static_cast<long long>(before);
    for (int i = i0; i < i1; ++i) {
      if (mask_allows(mask, i) && order_key(__fmul_rn(lg[i], inv_t)) == dk) {
        if (seen == tie_index) { sh.token = i; break; }
        ++seen;
      }
    }
  }
  __syncthreads();
  finish(sh.token >= 0 ? kSampleOk : kSampleInternal, sh.token);
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_sample_rows(const float* logits, long long ld, int rows, int vocab, const uint32_t* masks,
                                int mask_words, const ds41_sample_row* params, int* tokens, int* status, void* stream) {
  if (logits == nullptr || params == nullptr || tokens == nullptr || status == nullptr || rows <= 0 || vocab <= 0)
    return cudaErrorInvalidValue;
  if (masks != nullptr && mask_words != (vocab + 31) / 32) return cudaErrorInvalidValue;
  return launch_pdl(sample_rows_kernel, dim3(rows), dim3(kSampleThreads), 0, static_cast<cudaStream_t>(stream), logits,
                    ld, vocab, masks, mask_words, params, tokens, status);
}
