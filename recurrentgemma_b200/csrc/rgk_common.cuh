// Shared device helpers of librgk: dtype traits, 16-byte vector access, the rounding model of the
// bfloat16 mode, and the RG-LRU gate arithmetic (recurrentgemma torch/layers.py:338-353).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rgk {

// Workspace header (first 256 bytes of every workspace).
struct WsHeader {
  int status;          // 0, or RGK_ETIMEOUT once a bounded wait expired
  unsigned int ticket; // tile ticket of the look-back scan
  int pad[62];
};
static_assert(sizeof(WsHeader) == 256, "header is 256 bytes");

constexpr int kStatusTimeout = -7;
constexpr int kStatusBounds = -8;

// Range checks of computed indices for the -DRGK_CHECKS build (python -m recurrentgemma_b200.build
// --checks): an index outside its array raises WsHeader::status to kStatusBounds and the access is
// skipped - nothing traps, the kernel runs on.  In the normal build the macro is the bare condition
// `true`, so that `if (RGK_IN_RANGE(...)) access;` costs nothing.
#ifdef RGK_CHECKS
#define RGK_IN_RANGE(index, count, status_ptr) \
  rgk::index_in_range((long long)(index), (long long)(count), (status_ptr))
#else
#define RGK_IN_RANGE(index, count, status_ptr) true
#endif
__device__ __forceinline__ bool index_in_range(long long index, long long count, int* status) {
  if (index >= 0 && index < count) return true;
  if (status != nullptr) atomicExch(status, kStatusBounds);
  return false;
}

// ------------------------------------------------------------------------------------------------
// dtype traits.  A "pack" is 16 bytes: 4 float32 or 8 bfloat16 channels.
// ------------------------------------------------------------------------------------------------
template <typename T> struct Traits;
template <> struct Traits<float> {
  static constexpr int kPack = 4;
  static constexpr bool kBf16 = false;
};
template <> struct Traits<__nv_bfloat16> {
  static constexpr int kPack = 8;
  static constexpr bool kBf16 = true;
};

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Two floats -> packed bfloat16x2 (round to nearest even); `lo` lands in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Round a float to the nearest bfloat16 and widen it again.
__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

template <bool kBf16> __device__ __forceinline__ float rnd(float v) {
  if constexpr (kBf16) return round_bf16(v);
  return v;
}

// Unpack one 16-byte pack into floats / pack floats back (rounding in bfloat16 mode).
template <typename T> __device__ __forceinline__ void unpack(const uint4& v, float* f);
template <> __device__ __forceinline__ void unpack<float>(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
  f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& v, float* f) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
template <typename T> __device__ __forceinline__ uint4 pack(const float* f);
template <> __device__ __forceinline__ uint4 pack<float>(const float* f) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                    __float_as_uint(f[3]));
}
template <> __device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float* f) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                    pack_bf16x2(f[6], f[7]));
}

// Streaming 16-byte global access: activations are touched once, keep them out of L1.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};"
               :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// segment_pos == 0 for either index width.
__device__ __forceinline__ bool pos_is_zero(const void* pos, int is64, int64_t i) {
  return is64 ? (reinterpret_cast<const long long*>(pos)[i] == 0)
              : (reinterpret_cast<const int*>(pos)[i] == 0);
}

// ------------------------------------------------------------------------------------------------
// Scalar math.  The float32 mode uses the accurate library functions (the 1e-5 parity bar); the
// bfloat16 mode uses the SFU approximations, whose ~2 ulp float32 error is far below a bfloat16
// rounding step.
// ------------------------------------------------------------------------------------------------
template <bool kFast> __device__ __forceinline__ float exp_(float v) {
  if constexpr (kFast) return __expf(v);
  return expf(v);
}
template <bool kFast> __device__ __forceinline__ float sigmoid_(float z) {
  if constexpr (kFast) return __frcp_rn(1.0f + __expf(-z));
  return 1.0f / (1.0f + expf(-z));
}
template <bool kFast> __device__ __forceinline__ float sqrt_(float v) {
  if constexpr (kFast) {
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
  }
  return sqrtf(v);
}
// torch softplus defaults: beta 1, threshold 20.
__device__ __forceinline__ float softplus_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// gelu(approximate="tanh") written through the logistic function:
// 0.5 (1 + tanh(u)) = sigmoid(2u), u = sqrt(2/pi) (z + 0.044715 z^3).
template <bool kFast> __device__ __forceinline__ float gelu_tanh_(float z) {
  if constexpr (kFast) {
    const float u2 = 1.5957691216057308f * (z + 0.044715f * z * z * z);
    return z * sigmoid_<true>(u2);
  }
  const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  return 0.5f * z * (1.0f + tanhf(u));
}

// ------------------------------------------------------------------------------------------------
// Gate arithmetic of RGLRU.forward for one element (torch/layers.py:338-353).
//   c      conv output feeding the RG-LRU (tensor dtype)
//   zx, za float32 accumulators of the two block-diagonal projections (before the bias)
//   bx, ba gate biases; sp = softplus(a_param) already rounded to the tensor dtype
// Returns a (already multiplied by !reset, torch/layers.py:168) and the normalised input.
// In bfloat16 mode every tensor-level result is rounded exactly where torch rounds it.
// ------------------------------------------------------------------------------------------------
// kQuickF32 (float32 only): the sigmoids on the hardware exponential, a^2 as a * a and the
// hardware square root - a few 1e-7 of normalised error (measured 1.6e-6 -> 1.9e-6 at B2 T1024
// behind the 3xTF32 contraction, whose own error dominates), for the kernel whose epilogue this
// arithmetic bounds.  exp(log_a) itself stays on the accurate expf: a slow channel multiplies a
// into its state a thousand times.
template <bool kBf16, bool kQuickF32 = false>
__device__ __forceinline__ void gate_math(float c, float zx, float za, float bx, float ba, float sp,
                                          bool is_reset, float& a_out, float& xn_out) {
  constexpr bool kFast = kBf16;
  constexpr bool kFastAux = kBf16 || kQuickF32;
  const float gate_x = rnd<kBf16>(sigmoid_<kFastAux>(rnd<kBf16>(rnd<kBf16>(zx) + bx)));
  const float gate_a = rnd<kBf16>(sigmoid_<kFastAux>(rnd<kBf16>(rnd<kBf16>(za) + ba)));
  const float log_a = rnd<kBf16>((-8.0f * gate_a) * sp);
  const float e = exp_<kFast>(log_a);
  const float a = rnd<kBf16>(e);
  float a_square;
  if constexpr (kBf16) {
    a_square = round_bf16(e * e);          // exp(2 log_a) up to float32 rounding
  } else if constexpr (kQuickF32) {
    a_square = e * e;
  } else {
    a_square = expf(2.0f * log_a);
  }
  const float gated_x = rnd<kBf16>(c * gate_x);
  float mult = rnd<kBf16>(sqrt_<kFastAux>(rnd<kBf16>(1.0f - a_square)));
  if (is_reset) mult = 1.0f;
  a_out = is_reset ? 0.0f : a;
  xn_out = rnd<kBf16>(gated_x * mult);
}

}  // namespace rgk
