// RMSNorm over the last dimension (recurrentgemma torch/layers.py:65-73), the normalisation in
// front of the recurrent block (torch/modules.py:897-898):
//   var = mean(square(x), -1);  normed = x * rsqrt(var + eps);  out = normed * (scale + 1)
// HBM-bound: one warp owns a row, reads it once into registers (16-byte packs, lane-strided),
// reduces the sum of squares with shuffles and writes the row once.  In bfloat16 every tensor
// operation of the reference rounds: the squares, the mean, var + eps, the reciprocal square root,
// both products and scale + 1.  With an addend the kernel first forms x + addend (one rounding),
// writes that sum as well and normalises it: the residual add in front of a block's second norm
// (torch/modules.py:902-904) without a pass of its own.
#include "rgk_common.cuh"
#include "rgk_internal.h"

namespace rgk {
namespace {

constexpr int kNormWarps = 8;      // rows per block
constexpr int kMaxPacks = 32;      // 16-byte packs per lane: D <= 32 * 32 * pack elements

__device__ __forceinline__ uint32_t bf2mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf2add(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

template <typename T, int kPacks>   // kPacks: packs per lane this instantiation can hold
__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ addend, const T* __restrict__ scale,
               int64_t M, int D, float eps, T* __restrict__ sum_out, T* __restrict__ out) {
  constexpr int kPack = Traits<T>::kPack;
  constexpr bool kBf16 = Traits<T>::kBf16;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kNormWarps + (threadIdx.x >> 5);
  if (row >= M) return;
  const int packs = D / kPack;                 // packs in a row
  const T* xr = x + row * D;
  uint4 v[kPacks];
#pragma unroll
  for (int i = 0; i < kPacks; ++i) {
    const int pk = lane + 32 * i;
    v[i] = pk < packs ? ld_stream(xr + (int64_t)pk * kPack) : make_uint4(0u, 0u, 0u, 0u);
    if (addend != nullptr && pk < packs) {
      const uint4 w = ld_stream(addend + row * D + (int64_t)pk * kPack);
      if constexpr (kBf16) {
        v[i] = make_uint4(bf2add(v[i].x, w.x), bf2add(v[i].y, w.y), bf2add(v[i].z, w.z), bf2add(v[i].w, w.w));
      } else {
        v[i].x = __float_as_uint(__fadd_rn(__uint_as_float(v[i].x), __uint_as_float(w.x)));
        v[i].y = __float_as_uint(__fadd_rn(__uint_as_float(v[i].y), __uint_as_float(w.y)));
        v[i].z = __float_as_uint(__fadd_rn(__uint_as_float(v[i].z), __uint_as_float(w.z)));
        v[i].w = __float_as_uint(__fadd_rn(__uint_as_float(v[i].w), __uint_as_float(w.w)));
      }
      st_stream(sum_out + row * D + (int64_t)pk * kPack, v[i]);
    }
  }
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kPacks; ++i) {
    if constexpr (kBf16) {
      const uint32_t w[4] = {bf2mul(v[i].x, v[i].x), bf2mul(v[i].y, v[i].y), bf2mul(v[i].z, v[i].z),
                             bf2mul(v[i].w, v[i].w)};
#pragma unroll
      for (int k = 0; k < 4; ++k) sum += bf16_lo(w[k]) + bf16_hi(w[k]);
    } else {
      const float f[4] = {__uint_as_float(v[i].x), __uint_as_float(v[i].y), __uint_as_float(v[i].z),
                          __uint_as_float(v[i].w)};
#pragma unroll
      for (int k = 0; k < 4; ++k) sum = fmaf(f[k], f[k], sum);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float var = rnd<kBf16>(sum / (float)D);
  const float r = rnd<kBf16>(1.0f / sqrtf(rnd<kBf16>(var + eps)));
  T* orow = out + row * D;
  if constexpr (kBf16) {
    const uint32_t r2 = pack_bf16x2(r, r);
#pragma unroll
    for (int i = 0; i < kPacks; ++i) {
      const int pk = lane + 32 * i;
      if (pk < packs) {
        const uint4 sc = *reinterpret_cast<const uint4*>(scale + (int64_t)pk * kPack);
        constexpr uint32_t kOne = 0x3f803f80u;
        uint4 o;
        o.x = bf2mul(bf2mul(v[i].x, r2), bf2add(sc.x, kOne));
        o.y = bf2mul(bf2mul(v[i].y, r2), bf2add(sc.y, kOne));
        o.z = bf2mul(bf2mul(v[i].z, r2), bf2add(sc.z, kOne));
        o.w = bf2mul(bf2mul(v[i].w, r2), bf2add(sc.w, kOne));
        st_stream(orow + (int64_t)pk * kPack, o);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < kPacks; ++i) {
      const int pk = lane + 32 * i;
      if (pk < packs) {
        const float4 sc = *reinterpret_cast<const float4*>(scale + (int64_t)pk * kPack);
        uint4 o;
        o.x = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(v[i].x), r), __fadd_rn(sc.x, 1.0f)));
        o.y = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(v[i].y), r), __fadd_rn(sc.y, 1.0f)));
        o.z = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(v[i].z), r), __fadd_rn(sc.z, 1.0f)));
        o.w = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(v[i].w), r), __fadd_rn(sc.w, 1.0f)));
        st_stream(orow + (int64_t)pk * kPack, o);
      }
    }
  }
}

template <typename T>
cudaError_t launch_typed(const void* x, const void* addend, const void* scale, int64_t M, int64_t D,
                         float eps, void* sum_out, void* out, cudaStream_t s) {
  const int packs_per_lane = (int)((D / Traits<T>::kPack + 31) / 32);
  const unsigned grid = (unsigned)((M + kNormWarps - 1) / kNormWarps);
  const dim3 block(kNormWarps * 32);
#define RGK_NORM(P)                                                                           \
  rmsnorm_kernel<T, P><<<grid, block, 0, s>>>((const T*)x, (const T*)addend, (const T*)scale, M, (int)D, \
                                              eps, (T*)sum_out, (T*)out)
  if (packs_per_lane <= 4) RGK_NORM(4);
  else if (packs_per_lane <= 10) RGK_NORM(10);
  else if (packs_per_lane <= 16) RGK_NORM(16);
  else RGK_NORM(kMaxPacks);
#undef RGK_NORM
  return cudaGetLastError();
}

}  // namespace

bool rmsnorm_supported(int dtype, int64_t D) {
  const int pack = dtype ? 8 : 4;
  return D >= pack && D % pack == 0 && D <= (int64_t)kMaxPacks * 32 * pack;
}

cudaError_t launch_rmsnorm(const void* x, const void* scale, int64_t M, int64_t D, float eps,
                           int dtype, void* out, cudaStream_t s, const void* addend, void* sum_out) {
  if (M == 0) return cudaSuccess;
  return dtype ? launch_typed<__nv_bfloat16>(x, addend, scale, M, D, eps, sum_out, out, s)
               : launch_typed<float>(x, addend, scale, M, D, eps, sum_out, out, s);
}

}  // namespace rgk
