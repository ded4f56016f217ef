// CUDA-core block-diagonal projection (recurrentgemma torch/layers.py:127-137) with float32
// accumulation, and the same contraction for both RG-LRU gates fused with the gate arithmetic
// (torch/layers.py:338-353).  This is the float32-accurate path (tensor cores have no float32
// multiply) and the path for head widths the tcgen05 kernel does not cover.
//
// Tiling: a block computes 64 rows x 64 output channels of one head; each of its 256 threads owns
// a 4 x 4 patch.  K (the head width) is walked in slices of 16 staged through shared memory.
#include "rgk_common.cuh"
#include "rgk_internal.h"

namespace rgk {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, kThreads = 256;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// kGates == false: out = x w + b.      kGates == true: w/w2 are the input and a gate weights and the
// epilogue writes a (into out) and the normalised input (into out2).
template <typename T, bool kGates>
__global__ void __launch_bounds__(kThreads)
blockdiag_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                      const T* __restrict__ w2, const T* __restrict__ b2,
                      const T* __restrict__ a_param, const void* __restrict__ pos, int pos64,
                      int64_t M, int H, int bw, T* __restrict__ out, T* __restrict__ out2) {
  constexpr bool kBf16 = Traits<T>::kBf16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[kGates ? 2 : 1][BK][BN + 4];

  const int tid = threadIdx.x;
  const int tn = tid % 16, tm = tid / 16;
  const int n_tiles = (bw + BN - 1) / BN;
  const int h = blockIdx.y / n_tiles;
  const int n0 = (blockIdx.y % n_tiles) * BN;
  const int64_t m0 = (int64_t)blockIdx.x * BM;
  const int64_t E = (int64_t)H * bw;
  const T* wh = w + (int64_t)h * bw * bw;
  const T* wh2 = kGates ? w2 + (int64_t)h * bw * bw : nullptr;

  float acc[4][4], acc2[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = acc2[i][j] = 0.0f;

  for (int k0 = 0; k0 < bw; k0 += BK) {
    // A slice: 64 rows x 16 k.  Thread -> (row = i / 16, k = i % 16), 4 elements per thread.
#pragma unroll
    for (int r = 0; r < (BM * BK) / kThreads; ++r) {
      const int i = tid + r * kThreads;
      const int row = i / BK, kk = i % BK;
      const int64_t m = m0 + row;
      As[kk][row] = (m < M) ? to_f<T>(x[m * E + (int64_t)h * bw + k0 + kk]) : 0.0f;
    }
    // B slice: 16 k x 64 n.
#pragma unroll
    for (int r = 0; r < (BK * BN) / kThreads; ++r) {
      const int i = tid + r * kThreads;
      const int kk = i / BN, col = i % BN;
      const bool ok = (n0 + col) < bw;
      Bs[0][kk][col] = ok ? to_f<T>(wh[(int64_t)(k0 + kk) * bw + n0 + col]) : 0.0f;
      if constexpr (kGates)
        Bs[1][kk][col] = ok ? to_f<T>(wh2[(int64_t)(k0 + kk) * bw + n0 + col]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[4], bv2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][tm * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        bv[j] = Bs[0][kk][tn * 4 + j];
        if constexpr (kGates) bv2[j] = Bs[1][kk][tn * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
          if constexpr (kGates) acc2[i][j] = fmaf(av[i], bv2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + tm * 4 + i;
    if (m >= M) continue;
    bool is_reset = false;
    if constexpr (kGates) is_reset = pos_is_zero(pos, pos64, m);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn * 4 + j;
      if (n >= bw) continue;
      const int64_t e = (int64_t)h * bw + n;
      if constexpr (!kGates) {
        const float v = rnd<kBf16>(rnd<kBf16>(acc[i][j]) + to_f<T>(b[e]));
        out[m * E + e] = from_f<T>(v);
      } else {
        const float sp = rnd<kBf16>(softplus_(to_f<T>(a_param[e])));
        float a, xn;
        gate_math<kBf16>(to_f<T>(x[m * E + e]), acc[i][j], acc2[i][j], to_f<T>(b[e]),
                         to_f<T>(b2[e]), sp, is_reset, a, xn);
        out[m * E + e] = from_f<T>(a);
        out2[m * E + e] = from_f<T>(xn);
      }
    }
  }
}

}  // namespace

cudaError_t launch_blockdiag_linear_simt(const void* x, const void* w, const void* b, int64_t M,
                                         int H, int bw, int dtype, void* out, cudaStream_t s) {
  if (M == 0) return cudaSuccess;
  const int n_tiles = (bw + BN - 1) / BN;
  dim3 grid((unsigned)((M + BM - 1) / BM), (unsigned)(H * n_tiles));
  if (dtype) {
    using T_ = __nv_bfloat16;
    blockdiag_simt_kernel<T_, false><<<grid, kThreads, 0, s>>>(
        (const T_*)x, (const T_*)w, (const T_*)b, nullptr, nullptr, nullptr, nullptr, 0, M, H, bw,
        (T_*)out, nullptr);
  } else {
    blockdiag_simt_kernel<float, false><<<grid, kThreads, 0, s>>>(
        (const float*)x, (const float*)w, (const float*)b, nullptr, nullptr, nullptr, nullptr, 0, M,
        H, bw, (float*)out, nullptr);
  }
  return cudaGetLastError();
}

cudaError_t launch_gates_simt(const void* c, const void* pos, int pos64, const void* a_param,
                              const void* wx, const void* bx, const void* wa, const void* ba,
                              int64_t M, int H, int bw, int dtype, void* a_out, void* xn_out,
                              cudaStream_t s) {
  if (M == 0) return cudaSuccess;
  const int n_tiles = (bw + BN - 1) / BN;
  dim3 grid((unsigned)((M + BM - 1) / BM), (unsigned)(H * n_tiles));
  if (dtype) {
    using T_ = __nv_bfloat16;
    blockdiag_simt_kernel<T_, true><<<grid, kThreads, 0, s>>>(
        (const T_*)c, (const T_*)wx, (const T_*)bx, (const T_*)wa, (const T_*)ba,
        (const T_*)a_param, pos, pos64, M, H, bw, (T_*)a_out, (T_*)xn_out);
  } else {
    blockdiag_simt_kernel<float, true><<<grid, kThreads, 0, s>>>(
        (const float*)c, (const float*)wx, (const float*)bx, (const float*)wa, (const float*)ba,
        (const float*)a_param, pos, pos64, M, H, bw, (float*)a_out, (float*)xn_out);
  }
  return cudaGetLastError();
}

}  // namespace rgk
