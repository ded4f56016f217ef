// tcgen05 / TMEM wrappers, the shared-memory operand descriptor, and the RG-LRU gate arithmetic in
// packed bfloat16 (recurrentgemma torch/layers.py:338-353), shared by the tensor-core kernels.
#pragma once

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tma.cuh"

namespace rgk {

// Waits ask the hardware to suspend the thread for up to kWaitHintNs per attempt (it wakes when the
// barrier's phase completes), so a waiting thread issues an instruction only every so often; the
// number of attempts bounds the wait at about a second.
constexpr unsigned kWaitHintNs = 20000;
constexpr unsigned kWaitLimit = 1u << 16;

// Bounded wait.  Returns false (and raises the CTA's abort flag) when the limit is hit or another
// role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (unsigned i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity, kWaitHintNs)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// One lane of a converged warp.  Code that the whole warp runs with only the tcgen05 / TMA
// instructions under this predicate keeps its addresses and descriptors in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with operand A read from tensor memory: row = lane, a 32-bit column holds two
// consecutive K elements, so a K step of 16 bfloat16 is 8 columns.
__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 columns of this warp's 32 lanes <- 16 registers per thread
__device__ __forceinline__ void tc_st_32x16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
         "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]),
         "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_32x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand slice stored with the 128-byte swizzle:
// rows of 128 bytes, groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3ffffu) >> 4);        // start address, bits [0,14)
  d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset, bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                       // version
  d |= static_cast<uint64_t>(2) << 61;                       // SWIZZLE_128B
  return d;
}

// The same for rows of 64 bytes stored with the 64-byte swizzle: groups of 8 rows 512 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw64(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(4) << 61;                       // SWIZZLE_64B
  return d;
}

// Instruction descriptor of tcgen05.mma kind::f16: D float32, A and B bfloat16, both K-major.
constexpr uint32_t tc_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// packed bfloat16x2 arithmetic, each lane rounded to nearest even (what torch does per element)
__device__ __forceinline__ uint32_t bmul2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t badd2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bsub2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ float ex2f(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float rcpf(float v) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float sqrtf_approx(float v) {
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

// Gate arithmetic for two neighbouring channels (torch/layers.py:338-353), every tensor-level
// result rounded to bfloat16 where torch rounds it.
//   zx, za   float32 accumulators;  bx2, ba2 packed biases;  m8sp2 = packed -8 softplus(a_param)
//   c2       packed conv outputs;  returns packed a (reset-masked) and packed normalised input.
__device__ __forceinline__ void gate_pair(float zx0, float zx1, float za0, float za1, uint32_t bx2,
                                          uint32_t ba2, uint32_t m8sp2, uint32_t c2, bool is_reset,
                                          uint32_t& a2, uint32_t& xn2) {
  constexpr float kLog2e = 1.4426950408889634f;
  const uint32_t zx2 = badd2(pack_bf16x2(zx0, zx1), bx2);
  const uint32_t za2 = badd2(pack_bf16x2(za0, za1), ba2);
  // sigmoid(z) = 1 / (1 + 2^(-z log2 e)); the two gates of a channel share one reciprocal.
  // Arguments are clamped so that the product of the two denominators stays finite.
  const float ex0 = ex2f(fminf(-bf16_lo(zx2) * kLog2e, 60.0f));
  const float ex1 = ex2f(fminf(-bf16_hi(zx2) * kLog2e, 60.0f));
  const float ea0 = ex2f(fminf(-bf16_lo(za2) * kLog2e, 60.0f));
  const float ea1 = ex2f(fminf(-bf16_hi(za2) * kLog2e, 60.0f));
  const float dx0 = 1.0f + ex0, da0 = 1.0f + ea0, dx1 = 1.0f + ex1, da1 = 1.0f + ea1;
  const float r0 = rcpf(dx0 * da0), r1 = rcpf(dx1 * da1);
  const uint32_t gx2 = pack_bf16x2(r0 * da0, r1 * da1);
  const uint32_t ga2 = pack_bf16x2(r0 * dx0, r1 * dx1);
  // log_a = (-8 gate_a) softplus(a_param): the factor -8 is exact in bfloat16, so it is folded
  // into the per-channel constant.
  const uint32_t la2 = bmul2(ga2, m8sp2);
  const float e0 = ex2f(bf16_lo(la2) * kLog2e), e1 = ex2f(bf16_hi(la2) * kLog2e);
  a2 = pack_bf16x2(e0, e1);
  const uint32_t asq2 = pack_bf16x2(e0 * e0, e1 * e1);      // exp(2 log_a)
  const uint32_t om2 = bsub2(0x3f803f80u, asq2);            // 1 - a^2
  uint32_t mult2 = pack_bf16x2(sqrtf_approx(bf16_lo(om2)), sqrtf_approx(bf16_hi(om2)));
  if (is_reset) {
    mult2 = 0x3f803f80u;
    a2 = 0u;
  }
  xn2 = bmul2(bmul2(c2, gx2), mult2);
}

// ---- helpers shared by the fused RG-LRU kernels ------------------------------------------------

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int x, int y, int z, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
               :: "l"(map), "r"(x), "r"(y), "r"(z), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ uint32_t bmax2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
// tanh of both halves on the special-function unit; the result carries bfloat16 precision
__device__ __forceinline__ uint32_t btanh2(uint32_t a) {
  uint32_t r;
  asm("tanh.approx.bf16x2 %0, %1;" : "=r"(r) : "r"(a));
  return r;
}

// Gate arithmetic of ONE channel for two consecutive tokens (torch/layers.py:338-353), every
// tensor-level result rounded to bfloat16 where torch rounds it.
//   zx, za   float32 accumulators of the two tokens;  bx2, ba2, m8sp2: the channel's biases and
//   -8 softplus(a_param), each duplicated into both halves;  hbx2: half the input-gate bias.
// Returns packed a, x-gate and input multiplier, resets not yet applied.
// a = exp(log_a) and the input multiplier sqrt(1 - exp(2 log_a)) of a token pair, every rounding
// of the reference (torch/layers.py:343-350): both are functions of the bfloat16 value log_a alone.
__device__ __forceinline__ void a_mult_of_log_a(uint32_t la2, uint32_t& a2, uint32_t& mult2) {
  constexpr float kLog2e = 1.4426950408889634f;
  const float e0 = ex2f(bf16_lo(la2) * kLog2e), e1 = ex2f(bf16_hi(la2) * kLog2e);
  a2 = pack_bf16x2(e0, e1);
  const uint32_t om2 = bsub2(0x3f803f80u, pack_bf16x2(e0 * e0, e1 * e1));   // 1 - exp(2 log_a)
  mult2 = pack_bf16x2(sqrtf_approx(bf16_lo(om2)), sqrtf_approx(bf16_hi(om2)));
}

// The same from a table in shared memory, indexed by the magnitude bits of log_a (log_a <= 0).
// Up to 2^-11 both roundings give a = 1, multiplier 0 (the first entry); the table ends below 128,
// where a has long underflowed to 0 and the multiplier is 1: 18 binades x 128 values, one 32-bit
// entry {a, multiplier} each.  kLogAFloor: the most negative log_a the table covers.
constexpr uint32_t kLutBase = 0x3a00u;                 // bits of 2^-11
constexpr int kLutEntries = 0x4300 - 0x3a00;           // up to 128.0 (exclusive)
constexpr float kLogAFloor = -127.5f;
__device__ __forceinline__ uint32_t a_mult_entry(uint32_t index) {
  const uint32_t la = 0x8000u | (kLutBase + index);
  uint32_t a2, mult2;
  a_mult_of_log_a(la | (la << 16), a2, mult2);
  return (a2 & 0xffffu) | (mult2 << 16);
}
__device__ __forceinline__ void a_mult_lookup(uint32_t la2, const uint32_t* lut, uint32_t& a2,
                                              uint32_t& mult2) {
  // log_a is at most -2^-11 after the packed minimum (smaller magnitudes share the first entry),
  // and at least -127.5 because the per-channel factor -8 softplus(a_param) is clamped there when
  // it is computed (the gate is at most 1): the bits of each half, sign included, index the table
  // directly, relative to the bits of -2^-11.
  uint32_t m;
  asm("min.bf16x2 %0, %1, %2;" : "=r"(m) : "r"(la2), "r"(0x80008000u | kLutBase | (kLutBase << 16)));
  const uint32_t* base = lut - (0x8000u | kLutBase);
  const uint32_t e0 = base[m & 0xffffu], e1 = base[m >> 16];
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(a2) : "r"(e0), "r"(e1));
  asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(mult2) : "r"(e0), "r"(e1));
}

template <int kMath, bool kLut = false>
__device__ __forceinline__ void gate_tokens(float zx0, float zx1, float za0, float za1, uint32_t bx2,
                                            uint32_t ba2, uint32_t hbx2, uint32_t m8sp2, uint32_t& a2,
                                            uint32_t& gx2, uint32_t& mult2,
                                            const uint32_t* lut = nullptr) {
  constexpr float kNegLog2e = -1.4426950408889634f;
  uint32_t ga2;
  if constexpr (kMath == kMathExact) {
    constexpr uint32_t kFloor = 0xc1acc1acu;   // -21.5: the product of four denominators stays finite
    const uint32_t zx2 = bmax2(badd2(pack_bf16x2(zx0, zx1), bx2), kFloor);
    const uint32_t za2 = bmax2(badd2(pack_bf16x2(za0, za1), ba2), kFloor);
    const float dx0 = 1.0f + ex2f(bf16_lo(zx2) * kNegLog2e), dx1 = 1.0f + ex2f(bf16_hi(zx2) * kNegLog2e);
    const float da0 = 1.0f + ex2f(bf16_lo(za2) * kNegLog2e), da1 = 1.0f + ex2f(bf16_hi(za2) * kNegLog2e);
    const float p0 = dx0 * da0, p1 = dx1 * da1;
    const float r = rcpf(p0 * p1);
    const float r0 = r * p1, r1 = r * p0;      // 1 / p0, 1 / p1
    gx2 = pack_bf16x2(r0 * da0, r1 * da1);
    ga2 = pack_bf16x2(r0 * dx0, r1 * dx1);
  } else {
    constexpr uint32_t kFloor = 0xc226c226u;   // -41.5: the product of two denominators stays finite
    constexpr uint32_t kHalf2 = 0x3f003f00u;
    // round(0.5 zx + 0.5 bx) = 0.5 round(zx + bx): the reference's rounding of the biased value
    gx2 = bfma2(btanh2(bfma2(pack_bf16x2(zx0, zx1), kHalf2, hbx2)), kHalf2, kHalf2);
    const uint32_t za2 = bmax2(badd2(pack_bf16x2(za0, za1), ba2), kFloor);
    const float da0 = 1.0f + ex2f(bf16_lo(za2) * kNegLog2e), da1 = 1.0f + ex2f(bf16_hi(za2) * kNegLog2e);
    const float r = rcpf(da0 * da1);
    ga2 = pack_bf16x2(r * da1, r * da0);
  }
  // log_a = (-8 gate_a) softplus(a_param): -8 is exact in bfloat16 and folded into the constant
  const uint32_t la2 = bmul2(ga2, m8sp2);
  if constexpr (kLut) {
    a_mult_lookup(la2, lut, a2, mult2);
  } else {
    a_mult_of_log_a(la2, a2, mult2);
  }
}

// y2 * gelu_tanh(z2) for a token pair of one channel (torch/modules.py:289-291, 646): the gelu
// rounded to bfloat16, then the product rounded.
template <int kMath>
__device__ __forceinline__ uint32_t join_gelu2(uint32_t y2, uint32_t z2) {
  if constexpr (kMath == kMathExact) {
    constexpr float k0 = -1.5957691216057308f * 1.4426950408889634f;
    constexpr float k1 = k0 * 0.044715f;
    const float z0 = bf16_lo(z2), z1 = bf16_hi(z2);
    // gelu_tanh(z) = z sigmoid(2u) = z / (1 + 2^w); the exponent is capped so that the product of
    // the two denominators stays finite (the quotient is below 1e-18 |z| there either way)
    const float d0 = 1.0f + ex2f(fminf(z0 * fmaf(z0 * z0, k1, k0), 60.0f));
    const float d1 = 1.0f + ex2f(fminf(z1 * fmaf(z1 * z1, k1, k0), 60.0f));
    const float r = rcpf(d0 * d1);
    return bmul2(y2, pack_bf16x2(z0 * (r * d1), z1 * (r * d0)));
  } else {
    constexpr uint32_t kK0 = 0x3f4c3f4cu;      // sqrt(2/pi) = 0.7979 -> 0.796875
    constexpr uint32_t kK1 = 0x3d123d12u;      // 0.044715 sqrt(2/pi) = 0.035677 -> 0.035645
    constexpr uint32_t kHalf2 = 0x3f003f00u;
    const uint32_t u2 = bmul2(z2, bfma2(bmul2(z2, z2), kK1, kK0));
    const uint32_t hz2 = bmul2(z2, kHalf2);
    return bmul2(y2, bfma2(btanh2(u2), hz2, hz2));
  }
}

}  // namespace rgk
