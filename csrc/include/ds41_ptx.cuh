// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05
// (TMEM allocation, UMMA issue/commit, TMEM loads) and bounded waits.
//
// Every wait in this library is bounded: a wait that runs out records a status word
// in global memory and returns false, and the caller unwinds (frees TMEM, returns).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace ds41 {

// Status word layout written by kernels that give up on a wait.
enum StatusCode : int {
  kStatusOk = 0,
  kStatusMbarTimeout = 1,
  kStatusFlagTimeout = 2,
  kStatusBadArgument = 3,
};

// clock64 ticks after which a wait gives up (about one second at 2 GHz).
#ifndef DS41_WAIT_LIMIT_CYCLES
#define DS41_WAIT_LIMIT_CYCLES (2000000000ll)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Non-blocking probe (try_wait may suspend the thread for a hardware time slice before it answers "not yet"): for a
// thread that polls several barriers in turn.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait.  `status` points at an int[4] in global memory: {code, where, block, extra}.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ff) == 0) {
      if (clock64() - start > DS41_WAIT_LIMIT_CYCLES ||
          (status != nullptr && *reinterpret_cast<volatile int*>(status) != kStatusOk)) {
        if (status != nullptr && atomicCAS(status, kStatusOk, kStatusMbarTimeout) == kStatusOk) {
          status[1] = where;
          status[2] = static_cast<int>(blockIdx.x);
          status[3] = static_cast<int>(parity);
        }
        return false;
      }
    }
  }
  return true;
}

// Bounded spin on a 32-bit flag in (possibly peer) global memory until it is >= target.
__device__ __forceinline__ bool flag_wait_ge(const uint32_t* flag, uint32_t target, int* status, int where) {
  const long long start = clock64();
  uint32_t spins = 0;
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - target) >= 0) return true;
    if ((++spins & 0xff) == 0) {
      if (clock64() - start > DS41_WAIT_LIMIT_CYCLES ||
          (status != nullptr && *reinterpret_cast<volatile int*>(status) != kStatusOk)) {
        if (status != nullptr && atomicCAS(status, kStatusOk, kStatusFlagTimeout) == kStatusOk) {
          status[1] = where;
          status[2] = static_cast<int>(blockIdx.x);
          status[3] = static_cast<int>(v);
        }
        return false;
      }
    }
  }
}
// E2M1 (FP4) code of a value: magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6, round to nearest with ties to the even mantissa.
__device__ __forceinline__ uint32_t e2m1_code(float v) {
  const float a = fabsf(v);
  uint32_t c;
  // midpoints between representable magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6; ties go to the even mantissa
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.0f) c = 6;
  else c = 7;
  return c | (v < 0.f ? 8u : 0u);
}

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  const uint32_t m = code & 7u;
  const float a = m < 2u ? 0.5f * m : (m & 1u ? 1.5f : 1.0f) * static_cast<float>(1u << ((m >> 1) - 1u));
  return (code & 8u) ? -a : a;
}

// ------------------------------------------------------------------ FP4 index rows (E2M1 pairs + one UE8M0 scale per 32)
// A thread holds one pair of adjacent values; the 16 threads of a 32-value group (16 consecutive lanes, all active)
// agree on the scale ceil_pow2(max(amax, 6 * 2^-126) / 6) and each returns its packed byte (even value in the low
// nibble; saturating round-to-nearest-even on the E2M1 grid).  `mask` names the lanes that take part (taken with
// __activemask() where they are known to be converged, i.e. before any branch that splits a group).
// Reference: native/cuda/kernels/v41_compressor.cu:25-41.
__device__ __forceinline__ uint32_t fp4_group_pack(float a, float b, uint32_t* exponent_out, unsigned mask) {
  float m = fmaxf(fabsf(a), fabsf(b));
#pragma unroll
  for (int delta = 8; delta; delta >>= 1) m = fmaxf(m, __shfl_xor_sync(mask, m, delta, 16));
  m = fmaxf(m, 6.0f * 0x1p-126f);
  const uint32_t bits = __float_as_uint(m / 6.0f);
  const uint32_t exponent = (bits >> 23) + ((bits & 0x7fffffu) != 0 ? 1u : 0u);
  const float scale = __uint_as_float(exponent << 23);
  *exponent_out = exponent;
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(make_float2(a / scale, b / scale), __NV_E2M1, cudaRoundNearest));
}
// quantise and dequantise in place (the values an FP4 operand would carry)
__device__ __forceinline__ void fp4_group_qdq(float& a, float& b, unsigned mask) {
  uint32_t e;
  const uint32_t byte = fp4_group_pack(a, b, &e, mask);
  const float scale = __uint_as_float(e << 23);
  a = e2m1_value(byte & 15u) * scale;
  b = e2m1_value((byte >> 4) & 15u) * scale;
}

__device__ __forceinline__ void flag_store_release(uint32_t* flag, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}
__device__ __forceinline__ void flag_add_release(uint32_t* flag, uint32_t value) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

// ------------------------------------------------------------------ TMA
// Tiled loads into this CTA's shared memory; completion is signalled on `bar`.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// Untiled bulk copy global -> shared (16-byte aligned addresses, size multiple of 16).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Tiled store shared -> global (possibly a peer's memory), tracked by the issuing thread's bulk async-group.
// The innermost coordinate times the element size must be a multiple of 16 bytes and no coordinate may be negative.
__device__ __forceinline__ void tma_store_3d(const void* tmap, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most N of this thread's bulk groups may still be reading their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// at most N of this thread's bulk groups may be incomplete (writes not yet performed)
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ------------------------------------------------------------------ tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {         // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (8-row x 128 B atoms, consecutive atoms 1024 B apart).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;             // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;     // stride byte offset: 8 rows * 128 B
  d |= static_cast<uint64_t>(1) << 46;             // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;             // SWIZZLE_128B
  return d;
}
// Unswizzled K-major descriptor (used for scale-factor copies): 8x16 B core matrices.
__device__ __forceinline__ uint64_t umma_desc_plain(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// MN-major operand (the dimension that is NOT contracted is contiguous) in the 128-byte swizzle: 128-byte spans of 64
// bf16 along M/N, rows of the contracted dimension 128 bytes apart inside an 8-row atom; `mn_group_bytes` separates
// consecutive 64-element groups along M/N (leading byte offset), `k_group_bytes` consecutive 8-row groups along K
// (stride byte offset).
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t smem_addr, uint32_t mn_group_bytes,
                                                       uint32_t k_group_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(mn_group_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(k_group_bytes >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 / kind::tf32 / kind::f8f6f4 (dense, fp32 accumulate).
// a_fmt/b_fmt: f16 kinds 0=F16 1=BF16 2=TF32; f8f6f4 kinds 0=E4M3 1=E5M2 3=E2M3 4=E3M2 5=E2M1.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t m, uint32_t n, uint32_t a_fmt, uint32_t b_fmt) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Same with the B operand MN-major (bit 16), e.g. P x V where V is stored [key][dim] and the keys are contracted.
__host__ __device__ constexpr uint32_t umma_idesc_bmn(uint32_t m, uint32_t n, uint32_t a_fmt, uint32_t b_fmt) {
  return umma_idesc(m, n, a_fmt, b_fmt) | (1u << 16);
}
// Block-scaled kinds (mxf8f6f4 / mxf4 / mxf4nvf4): scale_fmt 0=E4M3 1=UE8M0; sf ids select the
// byte (scale_vec 1X) within the 32-bit TMEM scale column.
__host__ __device__ constexpr uint32_t umma_idesc_bs(uint32_t m, uint32_t n, uint32_t a_fmt, uint32_t b_fmt,
                                                     uint32_t scale_fmt, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (scale_fmt << 23) | ((m >> 4) << 24) |
         (a_sf_id << 29);
}

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Predicated forms for a warp that runs its issue loop convergently: every lane computes the (warp-uniform) operands
// and `issue` is true in the one lane that owns the instruction, so the descriptors never pass through a divergent
// region on their way to the tensor core.
__device__ __forceinline__ void umma_bf16_if(bool issue, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tc_commit_if(bool issue, uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(smem_u32(bar)), "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// e2m1 x e2m1 with one UE4M3 scale per 16 elements (NVFP4): K = 64 per instruction, four scales per row per operand.
__device__ __forceinline__ void umma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// smem (32 rows x 16 B) -> TMEM, replicated to the four 32-lane quadrants: scale-factor copy.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// predicated forms of the other kinds and of the scale-factor copy (see umma_bf16_if)
__device__ __forceinline__ void umma_f8_if(bool issue, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void umma_mxf8_if(bool issue, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %7, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem),
        "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void umma_nvf4_if(bool issue, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %7, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem),
        "r"(static_cast<uint32_t>(issue))
      : "memory");
}
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_if(bool issue, uint32_t taddr, uint64_t sdesc) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %2, 0;\n\t"
      "@q tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n\t}"
      ::"r"(taddr), "l"(sdesc), "r"(static_cast<uint32_t>(issue))
      : "memory");
}

// TMEM -> registers: 32 lanes x 32 consecutive 32-bit columns for the calling warp's lane quadrant.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// registers -> TMEM: the mirror image of tmem_ld_32x32 (complete after tmem_wait_st)
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr)
      : "memory");
}

// ------------------------------------------------------------------ small math helpers
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// Biased exponent of the smallest power of two >= x (UE8M0 scale, clamped to the finite range).
__device__ __forceinline__ uint32_t ue8m0_ceil_exp(float x) {
  x = fmaxf(x, 1.17549435e-38f);
  const uint32_t bits = __float_as_uint(x);
  uint32_t e = (bits >> 23) & 0xFF;
  if (bits & 0x7FFFFF) ++e;
  return e > 254 ? 254 : e;
}

}  // namespace ds41
