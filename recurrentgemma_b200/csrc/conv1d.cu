// Width-4 causal depthwise Conv1D of the recurrent block (recurrentgemma torch/layers.py:447-636),
// prefill and single-token decode form.  HBM-bound elementwise kernels: every thread owns one
// 16-byte pack of channels, rows are read once (plus a 3-row halo per time chunk).
#include "rgk_common.cuh"
#include "rgk_internal.h"

namespace rgk {
namespace {

constexpr int kConvRows = 24;     // output rows per thread (16: 64 us at B8 T4096 E2560, 24: 60, 28: 65)
constexpr int kConvThreads = 128; // packs (of 16 bytes) per block

// One tap: acc <- round(acc + round(x * w)); the first tap initialises acc (the reference starts
// from the Python float 0.0, torch/layers.py:483, 517).
template <bool kBf16, int kPack>
__device__ __forceinline__ void tap(float (&acc)[kPack], const float (&x)[kPack],
                                    const float (&w)[kPack], bool first) {
#pragma unroll
  for (int i = 0; i < kPack; ++i) {
    const float prod = rnd<kBf16>(__fmul_rn(x[i], w[i]));
    acc[i] = first ? prod : rnd<kBf16>(__fadd_rn(acc[i], prod));
  }
}

// 16-byte packs with the arithmetic of the tensor dtype: float32 lanes, or bfloat16 pairs whose
// products and sums are rounded to bfloat16 by the packed instructions themselves.
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf2_add(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <typename T> struct PackOps;
template <> struct PackOps<float> {
  static __device__ __forceinline__ uint4 mul(const uint4& a, const uint4& b) {
    return make_uint4(__float_as_uint(__fmul_rn(__uint_as_float(a.x), __uint_as_float(b.x))),
                      __float_as_uint(__fmul_rn(__uint_as_float(a.y), __uint_as_float(b.y))),
                      __float_as_uint(__fmul_rn(__uint_as_float(a.z), __uint_as_float(b.z))),
                      __float_as_uint(__fmul_rn(__uint_as_float(a.w), __uint_as_float(b.w))));
  }
  static __device__ __forceinline__ uint4 add(const uint4& a, const uint4& b) {
    return make_uint4(__float_as_uint(__fadd_rn(__uint_as_float(a.x), __uint_as_float(b.x))),
                      __float_as_uint(__fadd_rn(__uint_as_float(a.y), __uint_as_float(b.y))),
                      __float_as_uint(__fadd_rn(__uint_as_float(a.z), __uint_as_float(b.z))),
                      __float_as_uint(__fadd_rn(__uint_as_float(a.w), __uint_as_float(b.w))));
  }
  // x * 0 keeps the sign of x, as the reference's in-place masking does
  static __device__ __forceinline__ uint4 zero_like(const uint4& a) {
    return make_uint4(a.x & 0x80000000u, a.y & 0x80000000u, a.z & 0x80000000u, a.w & 0x80000000u);
  }
};
template <> struct PackOps<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 mul(const uint4& a, const uint4& b) {
    return make_uint4(bf2_mul(a.x, b.x), bf2_mul(a.y, b.y), bf2_mul(a.z, b.z), bf2_mul(a.w, b.w));
  }
  static __device__ __forceinline__ uint4 add(const uint4& a, const uint4& b) {
    return make_uint4(bf2_add(a.x, b.x), bf2_add(a.y, b.y), bf2_add(a.z, b.z), bf2_add(a.w, b.w));
  }
  static __device__ __forceinline__ uint4 zero_like(const uint4& a) {
    return make_uint4(a.x & 0x80008000u, a.y & 0x80008000u, a.z & 0x80008000u, a.w & 0x80008000u);
  }
};

template <typename T>
__global__ void __launch_bounds__(kConvThreads)
conv1d_prefill_kernel(const T* __restrict__ x, const void* __restrict__ pos, int pos64,
                      const T* __restrict__ w, const T* __restrict__ bias, int T_, int E,
                      T* __restrict__ out, T* __restrict__ cache_out) {
  constexpr int kPack = Traits<T>::kPack;
  using Ops = PackOps<T>;
  const int pack_idx = blockIdx.x * kConvThreads + threadIdx.x;
  const int e0 = pack_idx * kPack;
  if (e0 >= E) return;
  const int b = blockIdx.z;
  const int t_begin = blockIdx.y * kConvRows;
  const int64_t row0 = (int64_t)b * T_;

  // All rows this thread touches (3 halo rows + kConvRows), loaded back to back; rows outside the
  // sequence read a clamped address and are never used.
  uint4 xr[kConvRows + 3];
#pragma unroll
  for (int i = 0; i < kConvRows + 3; ++i) {
    const int t = min(max(t_begin - 3 + i, 0), T_ - 1);
    xr[i] = ld_stream(x + (row0 + t) * E + e0);
  }
  // nz bit i: row t_begin - 3 + i starts no document (rows outside the sequence count as set).
  unsigned nz = 0;
#pragma unroll
  for (int i = 0; i < kConvRows + 3; ++i) {
    const int t = t_begin - 3 + i;
    const bool inside = t >= 0 && t < T_;
    const bool z = pos_is_zero(pos, pos64, row0 + min(max(t, 0), T_ - 1));
    if (!(inside && z)) nz |= 1u << i;
  }
  uint4 wv[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) wv[k] = *reinterpret_cast<const uint4*>(w + (int64_t)k * E + e0);
  const uint4 bv = *reinterpret_cast<const uint4*>(bias + e0);

  // The common case - no document starts in the window, no sequence edge - is straight-line code:
  // four products and four sums per pack, nothing to decide per row.
  const bool plain = nz == ((1u << (kConvRows + 3)) - 1u) && t_begin >= 3 && t_begin + kConvRows <= T_;
  if (plain) {
#pragma unroll
    for (int r = 0; r < kConvRows; ++r) {
      const int i = r + 3;
      uint4 acc = Ops::mul(xr[i], wv[3]);
      acc = Ops::add(acc, Ops::mul(xr[i - 1], wv[2]));
      acc = Ops::add(acc, Ops::mul(xr[i - 2], wv[1]));
      acc = Ops::add(acc, Ops::mul(xr[i - 3], wv[0]));
      acc = Ops::add(acc, bv);
      st_stream(out + (row0 + t_begin + r) * E + e0, acc);
    }
    if (cache_out == nullptr || t_begin + kConvRows < T_) return;
  }
#pragma unroll
  for (int r = 0; r < kConvRows; ++r) {
    const int t = t_begin + r;
    if (!plain && t < T_) {
      const int i = r + 3;                       // index of row t inside xr
      // Tap s reaches row t-s and survives while rows t-s+1 .. t start no document.  A masked or
      // left-padded tap contributes round(acc + 0) = acc, so it is skipped
      // (torch/layers.py:487-517, 575-607).
      uint4 acc = Ops::mul(xr[i], wv[3]);
      const bool n0 = (nz >> i) & 1u, n1 = (nz >> (i - 1)) & 1u, n2 = (nz >> (i - 2)) & 1u;
      if (t >= 1 && n0) acc = Ops::add(acc, Ops::mul(xr[i - 1], wv[2]));
      if (t >= 2 && n0 && n1) acc = Ops::add(acc, Ops::mul(xr[i - 2], wv[1]));
      if (t >= 3 && n0 && n1 && n2) acc = Ops::add(acc, Ops::mul(xr[i - 3], wv[0]));
      acc = Ops::add(acc, bv);
      st_stream(out + (row0 + t) * E + e0, acc);
    }
  }

  // The block that owns the last row also writes the cache: rows T-3 .. T-1 of the input, each
  // multiplied by (0 or 1) for the document starts that follow it (torch/layers.py:497-508, 526).
  if (cache_out != nullptr && t_begin < T_ && t_begin + kConvRows >= T_) {
    const int il = T_ - 1 - t_begin + 3;         // index of row T-1 inside xr (>= 3)
    T* c = cache_out + (int64_t)b * 3 * E + e0;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int r = 0; r < kConvRows; ++r) {
      if (r + 3 == il) {
        const bool n0 = (nz >> (r + 3)) & 1u, n1 = (nz >> (r + 2)) & 1u;
        const uint4 x2 = xr[r + 1], x1 = xr[r + 2], x0 = xr[r + 3];   // rows T-3, T-2, T-1
        *reinterpret_cast<uint4*>(c) = (T_ >= 3) ? ((n0 && n1) ? x2 : Ops::zero_like(x2)) : zero;
        *reinterpret_cast<uint4*>(c + E) = (T_ >= 2) ? (n0 ? x1 : Ops::zero_like(x1)) : zero;
        *reinterpret_cast<uint4*>(c + 2 * (int64_t)E) = x0;
      }
    }
  }
}

// Only the cache a prefill returns (for callers that compute the convolution themselves): rows
// T-3 .. T-1 of the input, each multiplied by (0 or 1) for the document starts that follow it
// (torch/layers.py:497-508, 526).
template <typename T>
__global__ void __launch_bounds__(kConvThreads)
conv1d_cache_kernel(const T* __restrict__ x, const void* __restrict__ pos, int pos64, int T_, int E,
                    T* __restrict__ cache_out) {
  constexpr int kPack = Traits<T>::kPack;
  using Ops = PackOps<T>;
  const int e0 = (blockIdx.x * kConvThreads + threadIdx.x) * kPack;
  if (e0 >= E) return;
  const int b = blockIdx.y;
  const int64_t row0 = (int64_t)b * T_;
  // n0 / n1: rows T-1 / T-2 start no document
  const bool n0 = !pos_is_zero(pos, pos64, row0 + T_ - 1);
  const bool n1 = T_ >= 2 ? !pos_is_zero(pos, pos64, row0 + T_ - 2) : true;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  T* c = cache_out + (int64_t)b * 3 * E + e0;
  uint4 v2 = zero, v1 = zero;
  if (T_ >= 3) {
    const uint4 x2 = ld_stream(x + (row0 + T_ - 3) * E + e0);
    v2 = (n0 && n1) ? x2 : Ops::zero_like(x2);
  }
  if (T_ >= 2) {
    const uint4 x1 = ld_stream(x + (row0 + T_ - 2) * E + e0);
    v1 = n0 ? x1 : Ops::zero_like(x1);
  }
  *reinterpret_cast<uint4*>(c) = v2;
  *reinterpret_cast<uint4*>(c + E) = v1;
  *reinterpret_cast<uint4*>(c + 2 * (int64_t)E) = ld_stream(x + (row0 + T_ - 1) * E + e0);
}

template <typename T>
__global__ void __launch_bounds__(kConvThreads)
conv1d_decode_kernel(const T* x, const T* cache_in, const T* __restrict__ w,
                     const T* __restrict__ bias, int E, T* out, T* cache_out) {
  constexpr int kPack = Traits<T>::kPack;
  constexpr bool kBf16 = Traits<T>::kBf16;
  const int e0 = (blockIdx.x * kConvThreads + threadIdx.x) * kPack;
  if (e0 >= E) return;
  const int64_t b = blockIdx.y;
  float wv[kPack], xv[4][kPack], acc[kPack];
  const T* c = cache_in + b * 3 * E + e0;
#pragma unroll
  for (int k = 0; k < 3; ++k) unpack<T>(*reinterpret_cast<const uint4*>(c + (int64_t)k * E), xv[k]);
  unpack<T>(*reinterpret_cast<const uint4*>(x + b * E + e0), xv[3]);
  // Newest token first (torch/layers.py:491-517 with prompt_len = 3).
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    unpack<T>(*reinterpret_cast<const uint4*>(w + (int64_t)(3 - s) * E + e0), wv);
    tap<kBf16, kPack>(acc, xv[3 - s], wv, s == 0);
  }
  unpack<T>(*reinterpret_cast<const uint4*>(bias + e0), wv);
#pragma unroll
  for (int i = 0; i < kPack; ++i) acc[i] = rnd<kBf16>(__fadd_rn(acc[i], wv[i]));
  *reinterpret_cast<uint4*>(out + b * E + e0) = pack<T>(acc);
  if (cache_out != nullptr) {
    T* co = cache_out + b * 3 * E + e0;
#pragma unroll
    for (int k = 0; k < 3; ++k) *reinterpret_cast<uint4*>(co + (int64_t)k * E) = pack<T>(xv[k + 1]);
  }
}

}  // namespace

cudaError_t launch_conv1d_prefill(const void* x, const void* pos, int pos64, const void* w,
                                  const void* b, int64_t B, int64_t T, int64_t E, int dtype,
                                  void* out, void* cache_out, cudaStream_t s) {
  if (B == 0 || T == 0 || E == 0) return cudaSuccess;
  const int pack = dtype ? 8 : 4;
  dim3 grid((unsigned)((E / pack + kConvThreads - 1) / kConvThreads),
            (unsigned)((T + kConvRows - 1) / kConvRows), (unsigned)B);
  if (dtype) {
    using T_ = __nv_bfloat16;
    conv1d_prefill_kernel<T_><<<grid, kConvThreads, 0, s>>>(
        (const T_*)x, pos, pos64, (const T_*)w, (const T_*)b, (int)T, (int)E, (T_*)out,
        (T_*)cache_out);
  } else {
    conv1d_prefill_kernel<float><<<grid, kConvThreads, 0, s>>>(
        (const float*)x, pos, pos64, (const float*)w, (const float*)b, (int)T, (int)E, (float*)out,
        (float*)cache_out);
  }
  return cudaGetLastError();
}

cudaError_t launch_conv1d_cache(const void* x, const void* pos, int pos64, int64_t B, int64_t T,
                                int64_t E, int dtype, void* cache_out, cudaStream_t s) {
  if (B == 0 || T == 0 || E == 0 || cache_out == nullptr) return cudaSuccess;
  const int pack = dtype ? 8 : 4;
  dim3 grid((unsigned)((E / pack + kConvThreads - 1) / kConvThreads), (unsigned)B);
  if (dtype)
    conv1d_cache_kernel<__nv_bfloat16><<<grid, kConvThreads, 0, s>>>(
        (const __nv_bfloat16*)x, pos, pos64, (int)T, (int)E, (__nv_bfloat16*)cache_out);
  else
    conv1d_cache_kernel<float><<<grid, kConvThreads, 0, s>>>((const float*)x, pos, pos64, (int)T,
                                                            (int)E, (float*)cache_out);
  return cudaGetLastError();
}

cudaError_t launch_conv1d_decode(const void* x, const void* cache_in, const void* w, const void* b,
                                 int64_t B, int64_t E, int dtype, void* out, void* cache_out,
                                 cudaStream_t s) {
  if (B == 0 || E == 0) return cudaSuccess;
  const int pack = dtype ? 8 : 4;
  dim3 grid((unsigned)((E / pack + kConvThreads - 1) / kConvThreads), (unsigned)B);
  if (dtype) {
    using T_ = __nv_bfloat16;
    conv1d_decode_kernel<T_><<<grid, kConvThreads, 0, s>>>((const T_*)x, (const T_*)cache_in,
                                                         (const T_*)w, (const T_*)b, (int)E,
                                                         (T_*)out, (T_*)cache_out);
  } else {
    conv1d_decode_kernel<float><<<grid, kConvThreads, 0, s>>>(
        (const float*)x, (const float*)cache_in, (const float*)w, (const float*)b, (int)E,
        (float*)out, (float*)cache_out);
  }
  return cudaGetLastError();
}

}  // namespace rgk
