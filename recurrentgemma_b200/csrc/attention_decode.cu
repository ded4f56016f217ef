// Local attention for one new token per sequence against the ring-buffer cache
// (recurrentgemma torch/modules.py:437-476 with the cache branch, the mask of
// torch/modules.py:155-184 and the ring update of torch/modules.py:187-286), head dimension 256,
// one key/value head:
//   attn_decode_logits_kernel  logits of the N query heads against the W ring entries and the
//                              new key: contraction rounded to the activation dtype, scaled by
//                              head_dim^-1/2 (rounded again), entries outside the window marked;
//   attn_decode_values_kernel  float32 softmax over the W + 1 logits of a head, probabilities
//                              rounded, product with the ring's values and the new value, then
//                              the new key and value take their ring slot and num_tokens grows.
// Both are bandwidth work on the ring (2 W 256 elements per sequence), so they run on the CUDA
// cores: a warp reads a 256-element row as one pack per lane.
#include <math.h>

#include "rgk_common.cuh"
#include "rgk_internal.h"

namespace rgk {
namespace {

constexpr int kHdD = 256;
constexpr int kPerLane = kHdD / 32;        // 8 elements of a row per lane
constexpr float kMasked = -3.0e38f;        // marks a ring entry the query does not see

// This lane's 8 elements of a 256-element row.
template <typename T>
__device__ __forceinline__ void load_row(const T* row, int lane, float (&f)[kPerLane]) {
  if constexpr (Traits<T>::kBf16) {
    const uint4 v = ld_stream(row + lane * kPerLane);
    unpack<T>(v, f);
  } else {
    const uint4 v0 = ld_stream(row + lane * kPerLane), v1 = ld_stream(row + lane * kPerLane + 4);
    unpack<T>(v0, f);
    unpack<T>(v1, f + 4);
  }
}

// Ring slot j holds the latest position congruent to j (mod W) that is below nt, the number of
// tokens seen; the query, at position nt, sees positions nt - W .. nt (torch/modules.py:155-184).
// Once the ring is full every slot holds such a position; before that only slots below nt are
// filled.  So the visible slots are exactly j < nt.
__device__ __forceinline__ int visible_slots(int nt, int W) { return nt < W ? nt : W; }

// grid (B, splits): the warps of CTA (b, c) take entries 8 c + warp, + 8 splits, ... of the W ring
// rows followed by the new key (entry W).  logits: float [B, kN, W + 1].
template <typename T, int kN>
__global__ void __launch_bounds__(256)
attn_decode_logits_kernel(const T* __restrict__ q, const T* __restrict__ k_new,
                          const T* __restrict__ keys, const int* __restrict__ num_tokens, int W,
                          float* __restrict__ logits) {
  constexpr bool kBf16 = Traits<T>::kBf16;
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = num_tokens[b];
  const float scale = 0.0625f;                     // 256^-1/2
  float qf[kN][kPerLane];
#pragma unroll
  for (int n = 0; n < kN; ++n) load_row<T>(q + ((int64_t)b * kN + n) * kHdD, lane, qf[n]);
  float* lg = logits + (int64_t)b * kN * (W + 1);
  const int stride = gridDim.y * 8;
  const int n_vis = visible_slots(nt, W);
  for (int s = blockIdx.y * 8 + warp; s <= W; s += stride) {
    const bool self = s == W;
    if (!self && s >= n_vis) {
      if (lane < kN) lg[(int64_t)lane * (W + 1) + s] = kMasked;
      continue;
    }
    float kf[kPerLane];
    load_row<T>(self ? k_new + (int64_t)b * kHdD : keys + ((int64_t)b * W + s) * kHdD, lane, kf);
    float part[kN];
#pragma unroll
    for (int n = 0; n < kN; ++n) {
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) a = fmaf(qf[n][i], kf[i], a);
      part[n] = a;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int n = 0; n < kN; ++n) part[n] += __shfl_xor_sync(0xffffffffu, part[n], o);
    }
    // two tensor operations in the reference: the contraction, then the scaling
    float mine = 0.0f;
#pragma unroll
    for (int n = 0; n < kN; ++n)
      if (lane == n) mine = rnd<kBf16>(rnd<kBf16>(part[n]) * scale);
    if (lane < kN) lg[(int64_t)lane * (W + 1) + s] = mine;
  }
}

// grid (B, 4): CTA (b, dq) owns 64 of the 256 value columns.  Threads: warp w takes ring rows
// w, w + 8, ...; a lane holds two adjacent columns.  The probabilities of all kN heads of this
// sequence are first formed in shared memory (each CTA of a sequence repeats that small step).
template <typename T, int kN>
__global__ void __launch_bounds__(256)
attn_decode_values_kernel(const float* __restrict__ logits, const T* __restrict__ k_new,
                          const T* __restrict__ v_new, T* __restrict__ keys, T* __restrict__ values,
                          int* __restrict__ num_tokens, int W, int update, T* __restrict__ out) {
  constexpr bool kBf16 = Traits<T>::kBf16;
  extern __shared__ float s_p[];                   // [kN][W + 1] probabilities, then the partial sums
  __shared__ float s_red[8][kN];
  __shared__ float s_stat[2][kN];
  const int b = blockIdx.x, dq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = num_tokens[b];
  const int L = W + 1;
  const float* lg = logits + (int64_t)b * kN * L;
  // ---- softmax statistics of every head: maximum, then the sum of exponentials -----------------
  float mx[kN], sm[kN];
#pragma unroll
  for (int n = 0; n < kN; ++n) {
    float m = kMasked;
    for (int s = threadIdx.x; s < L; s += 256) m = fmaxf(m, lg[(int64_t)n * L + s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_red[warp][n] = m;
  }
  __syncthreads();
  if (threadIdx.x < kN) {
    float m = kMasked;
    for (int w = 0; w < 8; ++w) m = fmaxf(m, s_red[w][threadIdx.x]);
    s_stat[0][threadIdx.x] = m;
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < kN; ++n) {
    mx[n] = s_stat[0][n];
    float a = 0.0f;
    for (int s = threadIdx.x; s < L; s += 256) {
      const float v = lg[(int64_t)n * L + s];
      const float e = v > kMasked ? __expf(v - mx[n]) : 0.0f;
      s_p[n * L + s] = e;
      a += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    sm[n] = a;
  }
  __syncthreads();                                 // s_red is rewritten
#pragma unroll
  for (int n = 0; n < kN; ++n)
    if (lane == 0) s_red[warp][n] = sm[n];
  __syncthreads();
  if (threadIdx.x < kN) {
    float a = 0.0f;
    for (int w = 0; w < 8; ++w) a += s_red[w][threadIdx.x];
    s_stat[1][threadIdx.x] = a;
  }
  __syncthreads();
  // normalised probabilities, rounded to the activation dtype as the reference casts them
#pragma unroll
  for (int n = 0; n < kN; ++n) {
    const float inv = 1.0f / s_stat[1][n];
    for (int s = threadIdx.x; s < L; s += 256) s_p[n * L + s] = rnd<kBf16>(s_p[n * L + s] * inv);
  }
  __syncthreads();
  // ---- probabilities x values over this CTA's 64 columns ----------------------------------------
  // a lane holds 8 adjacent columns of one of the 4 rows its warp reads per instruction
  const int r4 = lane >> 3, c8 = (lane & 7) * 8;
  const int n_vis = visible_slots(nt, W);
  float acc[kN][8];
#pragma unroll
  for (int n = 0; n < kN; ++n)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[n][i] = 0.0f;
  auto row_of = [&](int s) {
    return s == W ? v_new + (int64_t)b * kHdD : values + ((int64_t)b * W + s) * kHdD;
  };
  auto load8 = [&](const T* p, float (&f)[8]) {
    if constexpr (kBf16) {
      unpack<T>(ld_stream(p), f);
    } else {
      unpack<T>(ld_stream(p), f);
      unpack<T>(ld_stream(p + 4), f + 4);
    }
  };
  // entries n_vis .. W - 1 are empty; entry W (the new value) is taken as if it were entry n_vis
  const int total = n_vis + 1;
#pragma unroll 1
  for (int e0 = warp * 4 + r4; e0 < total; e0 += 4 * 32) {
    float vf[4][8];
    int ss[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = e0 + 32 * u;
      ss[u] = e < total ? (e == n_vis ? W : e) : -1;
      if (ss[u] >= 0) load8(row_of(ss[u]) + dq * 64 + c8, vf[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (ss[u] < 0) continue;
#pragma unroll
      for (int n = 0; n < kN; ++n) {
        const float p = s_p[n * L + ss[u]];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[n][i] = fmaf(p, vf[u][i], acc[n][i]);
      }
    }
  }
  // the 4 rows of a warp, then the 8 warps
#pragma unroll
  for (int n = 0; n < kN; ++n)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      acc[n][i] += __shfl_xor_sync(0xffffffffu, acc[n][i], 8);
      acc[n][i] += __shfl_xor_sync(0xffffffffu, acc[n][i], 16);
    }
  __syncthreads();                                 // the probabilities are no longer needed
  float* s_acc = s_p;                              // [8 warps][kN][64]
  if (r4 == 0) {
#pragma unroll
    for (int n = 0; n < kN; ++n)
#pragma unroll
      for (int i = 0; i < 8; ++i) s_acc[(warp * kN + n) * 64 + c8 + i] = acc[n][i];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kN * 64; i += 256) {
    const int n = i / 64, c = i % 64;
    float a = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) a += s_acc[(w * kN + n) * 64 + c];
    out[((int64_t)b * kN + n) * kHdD + dq * 64 + c] = Traits<T>::kBf16 ? (T)__float2bfloat16(a) : (T)a;
  }
  // ---- the new token takes its ring slot (its 64 columns of both rows) --------------------------
  if (update) {
    const int slot = nt % W;
    if (threadIdx.x < 64) {
      const int c = dq * 64 + threadIdx.x;
      keys[((int64_t)b * W + slot) * kHdD + c] = k_new[(int64_t)b * kHdD + c];
      values[((int64_t)b * W + slot) * kHdD + c] = v_new[(int64_t)b * kHdD + c];
    }
  }
}

// num_tokens grows only after every CTA of the values kernel has read it.
__global__ void bump_tokens_kernel(int* num_tokens, int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) num_tokens[b] += 1;
}

template <typename T, int kN>
cudaError_t launch_decode_t(const void* q, const void* k_new, const void* v_new, void* keys,
                            void* values, int* num_tokens, int64_t B, int W, int update, void* out,
                            float* logits, cudaStream_t s) {
  const int splits = 8;
  attn_decode_logits_kernel<T, kN><<<dim3((unsigned)B, splits), 256, 0, s>>>(
      (const T*)q, (const T*)k_new, (const T*)keys, num_tokens, W, logits);
  const size_t a = (size_t)kN * (W + 1), r = (size_t)8 * kN * 64;
  const size_t smem = (a > r ? a : r) * sizeof(float);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(attn_decode_values_kernel<T, kN>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr_set = true;
  }
  attn_decode_values_kernel<T, kN><<<dim3((unsigned)B, 4), 256, smem, s>>>(
      logits, (const T*)k_new, (const T*)v_new, (T*)keys, (T*)values, num_tokens, W, update, (T*)out);
  if (update) bump_tokens_kernel<<<(unsigned)((B + 255) / 256), 256, 0, s>>>(num_tokens, (int)B);
  return cudaGetLastError();
}

}  // namespace

bool attention_decode_supported(int hd, int N, int W) {
  const bool heads = N == 1 || N == 2 || N == 4 || N == 8 || N == 10 || N == 16;
  // the probabilities of one sequence live in shared memory
  return hd == kHdD && heads && W >= 1 && (size_t)N * (W + 1) * sizeof(float) <= 200 * 1024;
}

size_t attention_decode_workspace_bytes(int64_t B, int N, int W) {
  return (((size_t)B * N * (W + 1) * sizeof(float)) + 255) & ~(size_t)255;
}

cudaError_t launch_attention_decode(const void* q, const void* k_new, const void* v_new, void* keys,
                                    void* values, int* num_tokens, int64_t B, int N, int W,
                                    int dtype, int update, void* out, void* ws, cudaStream_t s) {
  if (B == 0) return cudaSuccess;
  float* lg = reinterpret_cast<float*>(ws);
#define RGK_DEC(NN)                                                                              \
  case NN:                                                                                       \
    return dtype == 1 ? launch_decode_t<__nv_bfloat16, NN>(q, k_new, v_new, keys, values,        \
                                                           num_tokens, B, W, update, out, lg, s) \
                      : launch_decode_t<float, NN>(q, k_new, v_new, keys, values, num_tokens, B, \
                                                   W, update, out, lg, s)
  switch (N) {
    RGK_DEC(1); RGK_DEC(2); RGK_DEC(4); RGK_DEC(8); RGK_DEC(10); RGK_DEC(16);
    default: return cudaErrorInvalidValue;
  }
#undef RGK_DEC
}

}  // namespace rgk
