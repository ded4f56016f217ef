// Single-token step of the RG-LRU recurrence (recurrentgemma torch/layers.py:170-177): the new
// state is the unrounded float32 a h + x, the output its value in the activation dtype, optionally
// joined with the block's gelu branch (torch/modules.py:627-628, 646).
#include "rgk_common.cuh"
#include "rgk_internal.h"

namespace rgk {
namespace {

constexpr int kThreads = 128;

template <typename T, bool kMul>
__global__ void __launch_bounds__(kThreads)
decode_update_kernel(const T* __restrict__ a, const T* __restrict__ xn, const float* h_in,
                     const T* __restrict__ yb, int64_t n_packs, T* __restrict__ out, float* h_out) {
  constexpr int kPack = Traits<T>::kPack;
  constexpr bool kBf16 = Traits<T>::kBf16;
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n_packs) return;
  const int64_t off = i * kPack;
  float av[kPack], xv[kPack], hv[kPack], ov[kPack];
  unpack<T>(*reinterpret_cast<const uint4*>(a + off), av);
  unpack<T>(*reinterpret_cast<const uint4*>(xn + off), xv);
#pragma unroll
  for (int k = 0; k < kPack; k += 4) {
    const float4 h4 = *reinterpret_cast<const float4*>(h_in + off + k);
    hv[k] = h4.x; hv[k + 1] = h4.y; hv[k + 2] = h4.z; hv[k + 3] = h4.w;
  }
#pragma unroll
  for (int k = 0; k < kPack; ++k) {
    hv[k] = __fadd_rn(__fmul_rn(av[k], hv[k]), xv[k]);
    ov[k] = rnd<kBf16>(hv[k]);
  }
  if constexpr (kMul) {
    float mv[kPack];
    unpack<T>(*reinterpret_cast<const uint4*>(yb + off), mv);
#pragma unroll
    for (int k = 0; k < kPack; ++k) ov[k] = rnd<kBf16>(ov[k] * rnd<kBf16>(gelu_tanh_<kBf16>(mv[k])));
  }
  *reinterpret_cast<uint4*>(out + off) = pack<T>(ov);
#pragma unroll
  for (int k = 0; k < kPack; k += 4)
    *reinterpret_cast<float4*>(h_out + off + k) = make_float4(hv[k], hv[k + 1], hv[k + 2], hv[k + 3]);
}

}  // namespace

cudaError_t launch_decode_update(const void* a, const void* xn, const float* h_in, const void* yb,
                                 int64_t B, int64_t E, int dtype, void* out, float* h_out,
                                 cudaStream_t s) {
  if (B == 0 || E == 0) return cudaSuccess;
  const int64_t n_packs = B * E / (dtype ? 8 : 4);
  const unsigned grid = (unsigned)((n_packs + kThreads - 1) / kThreads);
#define RGK_DEC_LAUNCH(TYPE, MUL)                                                            \
  decode_update_kernel<TYPE, MUL><<<grid, kThreads, 0, s>>>(                                 \
      (const TYPE*)a, (const TYPE*)xn, h_in, (const TYPE*)yb, n_packs, (TYPE*)out, h_out)
  if (dtype) {
    if (yb) RGK_DEC_LAUNCH(__nv_bfloat16, true); else RGK_DEC_LAUNCH(__nv_bfloat16, false);
  } else {
    if (yb) RGK_DEC_LAUNCH(float, true); else RGK_DEC_LAUNCH(float, false);
  }
#undef RGK_DEC_LAUNCH
  return cudaGetLastError();
}

}  // namespace rgk
