// Width-4 causal depthwise Conv1D of the recurrent block (recurrentgemma torch/layers.py:447-636),
// prefill and single-token decode form.  HBM-bound elementwise kernels: every thread owns one
// 16-byte pack of channels, rows are read once (plus a 3-row halo per time chunk).
#include "rgk_common.cuh"
#include "rgk_internal.h"

namespace rgk {
namespace {

constexpr int kConvRows = 32;     // output rows per thread
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

template <typename T>
__global__ void __launch_bounds__(kConvThreads)
conv1d_prefill_kernel(const T* __restrict__ x, const void* __restrict__ pos, int pos64,
                      const T* __restrict__ w, const T* __restrict__ bias, int T_, int E,
                      T* __restrict__ out, T* __restrict__ cache_out) {
  constexpr int kPack = Traits<T>::kPack;
  constexpr bool kBf16 = Traits<T>::kBf16;
  const int pack_idx = blockIdx.x * kConvThreads + threadIdx.x;
  const int e0 = pack_idx * kPack;
  if (e0 >= E) return;
  const int b = blockIdx.z;
  const int t_begin = blockIdx.y * kConvRows;
  const int t_end = min(t_begin + kConvRows, T_);
  const int64_t row0 = (int64_t)b * T_;

  float wv[4][kPack], bv[kPack];
#pragma unroll
  for (int k = 0; k < 4; ++k) unpack<T>(*reinterpret_cast<const uint4*>(w + (int64_t)k * E + e0), wv[k]);
  unpack<T>(*reinterpret_cast<const uint4*>(bias + e0), bv);

  // Rolling window: xm1/xm2/xm3 = rows t-1, t-2, t-3; n1, n2 = "row t-1 / t-2 starts no document".
  float xm1[kPack], xm2[kPack], xm3[kPack], xc[kPack];
  bool n1 = true, n2 = true;
#pragma unroll
  for (int i = 0; i < kPack; ++i) xm1[i] = xm2[i] = xm3[i] = 0.0f;
  if (t_begin >= 1) {
    unpack<T>(ld_stream(x + (row0 + t_begin - 1) * E + e0), xm1);
    n1 = !pos_is_zero(pos, pos64, row0 + t_begin - 1);
  }
  if (t_begin >= 2) {
    unpack<T>(ld_stream(x + (row0 + t_begin - 2) * E + e0), xm2);
    n2 = !pos_is_zero(pos, pos64, row0 + t_begin - 2);
  }
  if (t_begin >= 3) unpack<T>(ld_stream(x + (row0 + t_begin - 3) * E + e0), xm3);

  bool n0 = true;
  for (int t = t_begin; t < t_end; ++t) {
    unpack<T>(ld_stream(x + (row0 + t) * E + e0), xc);
    n0 = !pos_is_zero(pos, pos64, row0 + t);
    float acc[kPack];
    tap<kBf16, kPack>(acc, xc, wv[3], true);
    // Tap s reaches row t-s and survives while rows t-s+1 .. t start no document.  A masked or
    // left-padded tap contributes round(acc + 0) = acc, so it is skipped.
    if (t >= 1 && n0) tap<kBf16, kPack>(acc, xm1, wv[2], false);
    if (t >= 2 && n0 && n1) tap<kBf16, kPack>(acc, xm2, wv[1], false);
    if (t >= 3 && n0 && n1 && n2) tap<kBf16, kPack>(acc, xm3, wv[0], false);
#pragma unroll
    for (int i = 0; i < kPack; ++i) acc[i] = rnd<kBf16>(__fadd_rn(acc[i], bv[i]));
    st_stream(out + (row0 + t) * E + e0, pack<T>(acc));
    if (t + 1 < t_end) {
#pragma unroll
      for (int i = 0; i < kPack; ++i) { xm3[i] = xm2[i]; xm2[i] = xm1[i]; xm1[i] = xc[i]; }
      n2 = n1; n1 = n0;
    }
  }

  // The block that owns the last row also writes the cache: rows T-3 .. T-1 of the input, each
  // multiplied by (0 or 1) for the document starts that follow it (torch/layers.py:497-508, 526).
  if (cache_out != nullptr && t_end == T_ && t_begin < T_) {
    // Here xc = row T-1, xm1 = row T-2, xm2 = row T-3; n0 = n[T-1], n1 = n[T-2].
    float r[kPack];
    T* c = cache_out + (int64_t)b * 3 * E + e0;
    {
      const float k = (T_ >= 3) ? ((n0 && n1) ? 1.0f : 0.0f) : 0.0f;
#pragma unroll
      for (int i = 0; i < kPack; ++i) r[i] = (T_ >= 3) ? xm2[i] * k : 0.0f;
      *reinterpret_cast<uint4*>(c) = pack<T>(r);
    }
    {
      const float k = n0 ? 1.0f : 0.0f;
#pragma unroll
      for (int i = 0; i < kPack; ++i) r[i] = (T_ >= 2) ? xm1[i] * k : 0.0f;
      *reinterpret_cast<uint4*>(c + E) = pack<T>(r);
    }
    *reinterpret_cast<uint4*>(c + 2 * (int64_t)E) = pack<T>(xc);
  }
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
