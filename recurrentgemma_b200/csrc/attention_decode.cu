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

constexpr int kSplits = 8;                 // CTAs per sequence in the logits kernel

// grid (B, kSplits): the warps of CTA (b, c) take entries 8 c + warp, + 8 kSplits, ... of the W ring
// rows followed by the new key (entry W).  logits: float [B, kN, W + 1]; stats: float2 [B, kSplits, kN] = the maximum of the CTA's
// visible logits of a head and the sum of exp(logit - maximum) over them.
template <typename T, int kN>
__global__ void __launch_bounds__(256)
attn_decode_logits_kernel(const T* __restrict__ q, const T* __restrict__ k_new,
                          const T* __restrict__ keys, const int* __restrict__ num_tokens, int W,
                          float* __restrict__ logits, float2* __restrict__ stats) {
  constexpr bool kBf16 = Traits<T>::kBf16;
  __shared__ float2 s_part[8][kN];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = num_tokens[b];
  const float scale = 0.0625f;                     // 256^-1/2
  float qf[kN][kPerLane];
#pragma unroll
  for (int n = 0; n < kN; ++n) load_row<T>(q + ((int64_t)b * kN + n) * kHdD, lane, qf[n]);
  float* lg = logits + (int64_t)b * kN * (W + 1);
  const int stride = gridDim.y * 8;
  const int n_vis = visible_slots(nt, W);
  float m_run = kMasked, l_run = 0.0f;             // lanes < kN: this warp's statistics of head `lane`
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
    if (lane < kN) {
      lg[(int64_t)lane * (W + 1) + s] = mine;
      const float m_new = fmaxf(m_run, mine);
      l_run = l_run * __expf(m_run - m_new) + __expf(mine - m_new);
      m_run = m_new;
    }
  }
  if (lane < kN) s_part[warp][lane] = make_float2(m_run, l_run);
  __syncthreads();
  if (threadIdx.x < kN) {
    float m = kMasked, l = 0.0f;
    for (int w = 0; w < 8; ++w) m = fmaxf(m, s_part[w][threadIdx.x].x);
    for (int w = 0; w < 8; ++w) {
      const float2 p = s_part[w][threadIdx.x];
      if (p.x > kMasked) l += p.y * __expf(p.x - m);
    }
    stats[((int64_t)b * kSplits + blockIdx.y) * kN + threadIdx.x] = make_float2(m, l);
  }
}

// grid (B, 4): CTA (b, dq) owns 64 of the 256 value columns.  A warp reads four ring rows per
// instruction: lane = (row of the four, 8 adjacent columns).  The 8 lanes of a row form that row's
// probabilities (head j and j + 8 in lane j) from the logits and the sequence's statistics, and
// pass them round by shuffles.
template <typename T, int kN>
__global__ void __launch_bounds__(256)
attn_decode_values_kernel(const float* __restrict__ logits, const float2* __restrict__ stats,
                          const T* __restrict__ k_new, const T* __restrict__ v_new,
                          T* __restrict__ keys, T* __restrict__ values,
                          int* __restrict__ num_tokens, int W, int update, T* __restrict__ out) {
  constexpr bool kBf16 = Traits<T>::kBf16;
  static_assert(kN <= 16, "two heads per lane of a row's eight");
  __shared__ float s_acc[8][kN][64];
  __shared__ float s_stat[2][16];                  // maximum and 1 / sum of every head
  const int b = blockIdx.x, dq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = num_tokens[b];
  const int L = W + 1;
  const float* lg = logits + (int64_t)b * kN * L;
  if (threadIdx.x < 16) {
    float m = kMasked, l = 0.0f;
    if (threadIdx.x < kN) {
      const float2* st = stats + (int64_t)b * kSplits * kN + threadIdx.x;
      for (int c = 0; c < kSplits; ++c) m = fmaxf(m, st[c * kN].x);
      for (int c = 0; c < kSplits; ++c) {
        const float2 p = st[c * kN];
        if (p.x > kMasked) l += p.y * __expf(p.x - m);
      }
    }
    s_stat[0][threadIdx.x] = m;
    s_stat[1][threadIdx.x] = l > 0.0f ? 1.0f / l : 0.0f;
  }
  __syncthreads();
  const int r4 = lane >> 3, j = lane & 7, c8 = j * 8;
  const float m_lo = s_stat[0][j], inv_lo = s_stat[1][j];
  const float m_hi = s_stat[0][j + 8], inv_hi = s_stat[1][j + 8];
  const int n_vis = visible_slots(nt, W);
  float acc[kN][8];
#pragma unroll
  for (int n = 0; n < kN; ++n)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[n][i] = 0.0f;
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
  // (the trip count is the same for every lane of a warp: the shuffles below need all of them)
#pragma unroll 1
  for (int base = warp * 4; base < total; base += 4 * 32) {
    float vf[4][8], p_lo[4], p_hi[4];
    int ss[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = base + r4 + 32 * u;
      ss[u] = e < total ? (e == n_vis ? W : e) : -1;
      if (ss[u] >= 0) {
        const T* row = ss[u] == W ? v_new + (int64_t)b * kHdD : values + ((int64_t)b * W + ss[u]) * kHdD;
        load8(row + dq * 64 + c8, vf[u]);
        p_lo[u] = j < kN ? lg[(int64_t)j * L + ss[u]] : kMasked;
        p_hi[u] = j + 8 < kN ? lg[(int64_t)(j + 8) * L + ss[u]] : kMasked;
      } else {
        p_lo[u] = p_hi[u] = kMasked;
#pragma unroll
        for (int i = 0; i < 8; ++i) vf[u][i] = 0.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      // normalised probabilities, rounded to the activation dtype as the reference casts them
      const float pl = p_lo[u] > kMasked ? rnd<kBf16>(__expf(p_lo[u] - m_lo) * inv_lo) : 0.0f;
      const float ph = p_hi[u] > kMasked ? rnd<kBf16>(__expf(p_hi[u] - m_hi) * inv_hi) : 0.0f;
#pragma unroll
      for (int n = 0; n < kN; ++n) {
        const float p = __shfl_sync(0xffffffffu, n < 8 ? pl : ph, (lane & 24) | (n & 7));
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
  if (r4 == 0) {
#pragma unroll
    for (int n = 0; n < kN; ++n)
#pragma unroll
      for (int i = 0; i < 8; ++i) s_acc[warp][n][c8 + i] = acc[n][i];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kN * 64; i += 256) {
    const int n = i / 64, c = i % 64;
    float a = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) a += s_acc[w][n][c];
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
                            float* logits, float2* stats, cudaStream_t s) {
  attn_decode_logits_kernel<T, kN><<<dim3((unsigned)B, kSplits), 256, 0, s>>>(
      (const T*)q, (const T*)k_new, (const T*)keys, num_tokens, W, logits, stats);
  attn_decode_values_kernel<T, kN><<<dim3((unsigned)B, 4), 256, 0, s>>>(
      logits, stats, (const T*)k_new, (const T*)v_new, (T*)keys, (T*)values, num_tokens, W, update,
      (T*)out);
  if (update) bump_tokens_kernel<<<(unsigned)((B + 255) / 256), 256, 0, s>>>(num_tokens, (int)B);
  return cudaGetLastError();
}

}  // namespace

bool attention_decode_supported(int hd, int N, int W) {
  const bool heads = N == 1 || N == 2 || N == 4 || N == 8 || N == 10 || N == 16;
  return hd == kHdD && heads && W >= 1;
}

// the logits [B, N, W + 1], then the per-CTA softmax statistics [B, kSplits, N]
static size_t decode_logits_bytes(int64_t B, int N, int W) {
  return (((size_t)B * N * (W + 1) * sizeof(float)) + 255) & ~(size_t)255;
}
size_t attention_decode_workspace_bytes(int64_t B, int N, int W) {
  return decode_logits_bytes(B, N, W) + ((((size_t)B * kSplits * N * sizeof(float2)) + 255) & ~(size_t)255);
}

cudaError_t launch_attention_decode(const void* q, const void* k_new, const void* v_new, void* keys,
                                    void* values, int* num_tokens, int64_t B, int N, int W,
                                    int dtype, int update, void* out, void* ws, cudaStream_t s) {
  if (B == 0) return cudaSuccess;
  float* lg = reinterpret_cast<float*>(ws);
  float2* st = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(ws) + decode_logits_bytes(B, N, W));
#define RGK_DEC(NN)                                                                              \
  case NN:                                                                                       \
    return dtype == 1 ? launch_decode_t<__nv_bfloat16, NN>(q, k_new, v_new, keys, values,        \
                                                           num_tokens, B, W, update, out, lg, st, s) \
                      : launch_decode_t<float, NN>(q, k_new, v_new, keys, values, num_tokens, B, \
                                                   W, update, out, lg, st, s)
  switch (N) {
    RGK_DEC(1); RGK_DEC(2); RGK_DEC(4); RGK_DEC(8); RGK_DEC(10); RGK_DEC(16);
    default: return cudaErrorInvalidValue;
  }
#undef RGK_DEC
}

}  // namespace rgk
