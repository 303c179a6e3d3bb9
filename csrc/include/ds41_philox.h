// Philox4x32-10 counter-based generator, shared by the host oracle and the device kernels.
// counter = {offset_lo, offset_hi, subsequence_lo, subsequence_hi}, key = {seed_lo, seed_hi}: a draw is a pure function
// of (seed, subsequence, offset), so a request that owns a subsequence can replay or skip draws freely.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define DS41_HD __host__ __device__ __forceinline__
#else
#define DS41_HD inline
#endif

namespace ds41 {

struct Philox4 {
  uint32_t v[4];
};

DS41_HD uint32_t philox_mulhi(uint32_t a, uint32_t b) {
  return static_cast<uint32_t>((static_cast<uint64_t>(a) * static_cast<uint64_t>(b)) >> 32);
}

DS41_HD Philox4 philox4x32_10(uint64_t seed, uint64_t subsequence, uint64_t offset) {
  uint32_t c0 = static_cast<uint32_t>(offset), c1 = static_cast<uint32_t>(offset >> 32);
  uint32_t c2 = static_cast<uint32_t>(subsequence), c3 = static_cast<uint32_t>(subsequence >> 32);
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = philox_mulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = philox_mulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return Philox4{{c0, c1, c2, c3}};
}

// uniform in (0, 1): 23 bits plus a half step, exactly representable in fp32, never 0 or 1
DS41_HD float philox_uniform(uint32_t bits) { return (static_cast<float>(bits >> 9) + 0.5f) * (1.0f / 8388608.0f); }

}  // namespace ds41
