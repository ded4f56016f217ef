// The two ends of the model around the residual blocks (recurrentgemma torch/modules.py:945-1003,
// torch/sampler.py:126-135):
//   embed_kernel   Embedder.encode: out[m, :] = table[tokens[m], :] * scale, one rounding in
//                  bfloat16 (the reference multiplies by sqrt(width) cast to bfloat16; the caller
//                  passes that constant, or 1);
//   argmax_kernel  greedy sampling: the index of the first maximum of each row of the logits;
//   geglu_bias_kernel  the element-wise part of MLPBlock.forward for a decode step, where the two
//                  halves of ffw_up come from a library contraction (torch/layers.py:700-703,
//                  torch/modules.py:749-751): gelu(up[0] + b[0]) * (up[1] + b[1]), each of the four
//                  tensor operations rounded.
#include "rgk_common.cuh"
#include "rgk_internal.h"

namespace rgk {
namespace {

// One warp per 16-byte pack column group: a block of 256 threads copies one row.
template <typename T>
__global__ void embed_kernel(const void* __restrict__ tokens, int tokens64, const T* __restrict__ table,
                             int64_t M, int64_t V, int64_t D, float scale, T* __restrict__ out) {
  constexpr int kPer = 16 / (int)sizeof(T);
  const int64_t m = blockIdx.x;
  if (m >= M) return;
  int64_t tok = tokens64 ? (int64_t)reinterpret_cast<const long long*>(tokens)[m]
                         : (int64_t)reinterpret_cast<const int*>(tokens)[m];
  // an index outside the table cannot be reported from here; it reads the nearest row
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  const T* src = table + tok * D;
  T* dst = out + m * D;
  const int packs = (int)(D / kPer);
  for (int p = threadIdx.x; p < packs; p += blockDim.x) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + (int64_t)p * kPer);
    float f[kPer];
    unpack<T>(v, f);
#pragma unroll
    for (int i = 0; i < kPer; ++i) f[i] *= scale;
    *reinterpret_cast<uint4*>(dst + (int64_t)p * kPer) = pack<T>(f);
  }
}

// One block per row.  Each thread keeps the first maximum of the packs it visits (its indices
// ascend, so "greater than" keeps the first); ties between threads go to the smaller index.
template <typename T>
__global__ void argmax_kernel(const T* __restrict__ x, int64_t M, int64_t V, int* __restrict__ out) {
  constexpr int kPer = 16 / (int)sizeof(T);
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  const int64_t m = blockIdx.x;
  if (m >= M) return;
  const T* row = x + m * V;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  // rows are 16-byte aligned only when V is a multiple of the pack width
  const int packs = V % kPer == 0 ? (int)(V / kPer) : 0;
  for (int p = threadIdx.x; p < packs; p += blockDim.x) {
    const uint4 v = ld_stream(row + (int64_t)p * kPer);
    float f[kPer];
    unpack<T>(v, f);
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      if (f[i] > best || best_i == 0x7fffffff) { best = f[i]; best_i = p * kPer + i; }
    }
  }
  for (int i = packs * kPer + threadIdx.x; i < V; i += blockDim.x) {   // a ragged tail
    const float f = static_cast<float>(row[i]);
    if (f > best || best_i == 0x7fffffff) { best = f; best_i = i; }
  }
  auto better = [](float a, int ai, float b, int bi) { return a > b || (a == b && ai < bi); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_down_sync(0xffffffffu, best, o);
    const int oi = __shfl_down_sync(0xffffffffu, best_i, o);
    if (oi != 0x7fffffff && (best_i == 0x7fffffff || better(ov, oi, best, best_i))) { best = ov; best_i = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? s_val[lane] : -INFINITY;
    best_i = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_down_sync(0xffffffffu, best, o);
      const int oi = __shfl_down_sync(0xffffffffu, best_i, o);
      if (oi != 0x7fffffff && (best_i == 0x7fffffff || better(ov, oi, best, best_i))) { best = ov; best_i = oi; }
    }
    if (lane == 0) out[m] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

// up [2, M, X], bias [2, X] -> out [M, X]; one 16-byte pack per thread.
template <typename T>
__global__ void geglu_bias_kernel(const T* __restrict__ up, const T* __restrict__ bias, int64_t M,
                                  int64_t X, T* __restrict__ out) {
  constexpr int kPer = 16 / (int)sizeof(T);
  constexpr bool kBf16 = Traits<T>::kBf16;
  const int64_t packs_row = X / kPer;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * packs_row) return;
  const int64_t col = (idx % packs_row) * kPer, off = (idx / packs_row) * X + col;
  float g[kPer], v[kPer], bg[kPer], bv[kPer], o[kPer];
  unpack<T>(ld_stream(up + off), g);
  unpack<T>(ld_stream(up + M * X + off), v);
  unpack<T>(*reinterpret_cast<const uint4*>(bias + col), bg);
  unpack<T>(*reinterpret_cast<const uint4*>(bias + X + col), bv);
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const float gate = rnd<kBf16>(g[i] + bg[i]), value = rnd<kBf16>(v[i] + bv[i]);
    o[i] = rnd<kBf16>(gelu_tanh_<kBf16>(gate)) * value;
  }
  *reinterpret_cast<uint4*>(out + off) = pack<T>(o);
}

}  // namespace

cudaError_t launch_geglu_bias(const void* up, const void* bias, int64_t M, int64_t X, int dtype,
                              void* out, cudaStream_t s) {
  if (M == 0) return cudaSuccess;
  const int per = dtype == 1 ? 8 : 4;
  const int64_t n = M * (X / per);
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dtype == 1)
    geglu_bias_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)up,
                                                         (const __nv_bfloat16*)bias, M, X,
                                                         (__nv_bfloat16*)out);
  else
    geglu_bias_kernel<float><<<grid, 256, 0, s>>>((const float*)up, (const float*)bias, M, X,
                                                  (float*)out);
  return cudaGetLastError();
}

cudaError_t launch_embed(const void* tokens, int tokens64, const void* table, int64_t M, int64_t V,
                         int64_t D, float scale, int dtype, void* out, cudaStream_t s) {
  if (M == 0) return cudaSuccess;
  if (M >= ((int64_t)1 << 31)) return cudaErrorInvalidValue;
  if (dtype == 1)
    embed_kernel<__nv_bfloat16><<<(unsigned)M, 256, 0, s>>>(
        tokens, tokens64, (const __nv_bfloat16*)table, M, V, D, scale, (__nv_bfloat16*)out);
  else
    embed_kernel<float><<<(unsigned)M, 256, 0, s>>>(tokens, tokens64, (const float*)table, M, V, D,
                                                    scale, (float*)out);
  return cudaGetLastError();
}

cudaError_t launch_argmax(const void* x, int64_t M, int64_t V, int dtype, int* out, cudaStream_t s) {
  if (M == 0) return cudaSuccess;
  if (M >= ((int64_t)1 << 31) || V >= ((int64_t)1 << 31)) return cudaErrorInvalidValue;
  if (dtype == 1)
    argmax_kernel<__nv_bfloat16><<<(unsigned)M, 512, 0, s>>>((const __nv_bfloat16*)x, M, V, out);
  else
    argmax_kernel<float><<<(unsigned)M, 512, 0, s>>>((const float*)x, M, V, out);
  return cudaGetLastError();
}

}  // namespace rgk
