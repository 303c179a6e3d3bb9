// Engram table conversion on the CPU: FP8 rows (E4M3 payload + UE8M0 scale per 32) -> NVFP4 rows (E2M1 pairs +
// E4M3 scale per 16 + one fp32 scale per table), without ever holding a decoded table.
//
//   pass 1  ds41_ple_scan     : largest magnitude of a block of records (NaN if a payload or scale byte encodes NaN)
//           global = amax / (6 * 448)
//   pass 2  ds41_ple_convert  : for every group of 16 values
//               block scale  s = e4m3_rne(clamp(group amax / (6 * global), 2^-9, 448)), 1.0 for an all-zero group
//               code         q = e2m1_rne(|v| / (s * global)), ties to the even code, sign taken from the source byte
//                                (a source zero stays +0: the recipe's sign test is `weight < 0`)
//             output record = dim/2 payload bytes (even element in the low nibble) followed by dim/16 scale bytes.
// Both passes take any contiguous run of records, so a driver can stream a table through them in bounded chunks and
// resume after a stop; the work is split over `threads` host threads by record.
// The arithmetic is the weight-only NVFP4 recipe (table amax -> fp32 scale, group amax -> E4M3 scale, round to nearest
// even) that the reference applies to its Engram tables: quantization/ple_nvfp4_cpu.cpp:29-82 and
// quantization/FP4PLE_PLAN.md of the reference.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

struct E4M3Table {
  float v[128];
  E4M3Table() {
    for (int c = 0; c < 128; ++c) {
      const int e = c >> 3, m = c & 7;
      v[c] = e ? std::ldexp(static_cast<float>(8 + m), e - 10) : std::ldexp(static_cast<float>(m), -9);
    }
    v[127] = std::numeric_limits<float>::quiet_NaN();
  }
};
const E4M3Table kE4M3;

inline float ue8m0(uint8_t e) { return std::ldexp(1.0f, static_cast<int>(e) - 127); }

// round to nearest even E4M3 code of x clamped to [2^-9, 448]
inline uint8_t e4m3_rne(float x) {
  x = std::min(std::max(x, std::ldexp(1.0f, -9)), 448.0f);
  if (x < std::ldexp(1.0f, -6)) return static_cast<uint8_t>(std::nearbyint(std::ldexp(x, 9)));   // 8 = smallest normal
  int e;
  const float f = std::frexp(x, &e);                   // x = f * 2^e, f in [0.5, 1)
  int m = static_cast<int>(std::nearbyint(std::ldexp(f, 4))) - 8;     // mantissa steps of 1/8 above 1.0
  int ex = e - 1 + 7;
  if (m == 8) { m = 0; ++ex; }
  const int code = (ex << 3) | m;
  return static_cast<uint8_t>(std::min(code, 0x7e));
}

// E2M1 magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6; a tie goes to the even code
inline uint8_t e2m1_rne(float x) {
  static const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  uint8_t c = 0;
  while (c < 7 && (x > mid[c] || (x == mid[c] && (c & 1)))) ++c;
  return c;
}

template <class F>
void split(uint64_t rows, int threads, F&& body) {
  threads = std::max(1, std::min<int>(threads, static_cast<int>(std::min<uint64_t>(rows, 256))));
  if (threads == 1) { body(0, uint64_t{0}, rows); return; }
  std::vector<std::thread> pool;
  const uint64_t per = (rows + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    const uint64_t lo = std::min(rows, per * t), hi = std::min(rows, lo + per);
    pool.emplace_back([&body, t, lo, hi] { body(t, lo, hi); });
  }
  for (auto& th : pool) th.join();
}

bool bad_geometry(const void* src, uint64_t rows, int dim, int src_row_bytes) {
  return src == nullptr || rows == 0 || dim <= 0 || (dim & 31) || src_row_bytes < dim + dim / 32;
}

}  // namespace

extern "C" {

// 0 = ok, 1 = bad arguments, 2 = the records hold a NaN (amax is NaN then).
int ds41_ple_scan(const uint8_t* src, uint64_t rows, int dim, int src_row_bytes, int threads, float* amax) {
  if (bad_geometry(src, rows, dim, src_row_bytes) || amax == nullptr) return 1;
  std::vector<float> best(256, 0.0f);
  std::vector<int> nan(256, 0);
  split(rows, threads, [&](int t, uint64_t lo, uint64_t hi) {
    float a = 0.0f;
    int bad = 0;
    for (uint64_t r = lo; r < hi; ++r) {
      const uint8_t* rec = src + r * src_row_bytes;
      for (int g = 0; g < dim / 32; ++g) {
        unsigned top = 0;
        for (int j = 0; j < 32; ++j) top = std::max<unsigned>(top, rec[g * 32 + j] & 127u);
        const uint8_t e = rec[dim + g];
        if (top == 127 || e == 255) { bad = 1; continue; }
        if (top) a = std::max(a, kE4M3.v[top] * ue8m0(e));
      }
    }
    best[t] = a;
    nan[t] = bad;
  });
  float a = 0.0f;
  int bad = 0;
  for (int t = 0; t < 256; ++t) { a = std::max(a, best[t]); bad |= nan[t]; }
  *amax = bad ? std::numeric_limits<float>::quiet_NaN() : a;
  return bad ? 2 : 0;
}

float ds41_ple_global_scale(float amax) { return amax / (6.0f * 448.0f); }

// 0 = ok, 1 = bad arguments.
int ds41_ple_convert(const uint8_t* src, uint64_t rows, int dim, int src_row_bytes, float global, uint8_t* dst,
                     int dst_row_bytes, int threads) {
  if (bad_geometry(src, rows, dim, src_row_bytes) || dst == nullptr || dst_row_bytes < dim / 2 + dim / 16 ||
      !std::isfinite(global) || global <= 0.0f)
    return 1;
  split(rows, threads, [&](int, uint64_t lo, uint64_t hi) {
    float v[16];
    for (uint64_t r = lo; r < hi; ++r) {
      const uint8_t* rec = src + r * src_row_bytes;
      uint8_t* out = dst + r * dst_row_bytes;
      if (dst_row_bytes > dim / 2 + dim / 16) std::memset(out + dim / 2 + dim / 16, 0, dst_row_bytes - dim / 2 - dim / 16);
      for (int g = 0; g < dim / 16; ++g) {
        const float es = ue8m0(rec[dim + g / 2]);
        float top = 0.0f;
        for (int j = 0; j < 16; ++j) {
          v[j] = kE4M3.v[rec[g * 16 + j] & 127] * es;
          top = std::max(top, v[j]);
        }
        const uint8_t sc = top > 0.0f ? e4m3_rne(top / (6.0f * global)) : e4m3_rne(1.0f);
        out[dim / 2 + g] = sc;
        const float divisor = kE4M3.v[sc] * global;
        for (int j = 0; j < 8; ++j) {
          uint8_t pair = 0;
          for (int h = 0; h < 2; ++h) {
            const uint8_t b = rec[g * 16 + 2 * j + h];
            uint8_t c = e2m1_rne(v[2 * j + h] / divisor);
            if ((b & 128) && (b & 127)) c |= 8;
            pair |= static_cast<uint8_t>(c << (4 * h));
          }
          out[g * 8 + j] = pair;
        }
      }
    }
  });
  return 0;
}

}  // extern "C"
