// Local attention for one new token per sequence against the ring-buffer cache
// (recurrentgemma torch/modules.py:437-476 with the cache branch, the mask of
// torch/modules.py:155-184 and the ring update of torch/modules.py:187-286), head dimension 256,
// one key/value head:
//   attn_decode_logits_kernel    logits of the N query heads against the W ring entries and the
//                                new key: contraction rounded to the activation dtype, scaled by
//                                head_dim^-1/2 (rounded again); per CTA the softmax statistics;
//   attn_decode_values_kernel    probabilities (float32 softmax over the W + 1 logits of a head,
//                                rounded) times the ring's values and the new value, a partial sum
//                                per CTA;
//   attn_decode_finish_kernel    sum of the partials, rounded; then the new key and value take
//                                their ring slot and num_tokens grows.
// All three are bandwidth work on the ring (2 W 256 elements per sequence) and run on the CUDA
// cores.  A warp reads a 256-element row as one 16-byte pack per lane and has the loads of a whole
// batch of rows in flight before it uses the first: with 16 CTAs per sequence that is several MB
// in flight, which a ring walked row by row does not reach.
#include <math.h>

#include "rgk_common.cuh"
#include "rgk_internal.h"

namespace rgk {
namespace {

constexpr int kHdD = 256;
constexpr int kPerLane = kHdD / 32;        // 8 elements of a row per lane
constexpr float kMasked = -3.0e38f;        // "no logit yet" in the running maxima
constexpr int kSplits = 16;                // CTAs per sequence in the logits and values kernels
constexpr int kHeadPad = 16;               // heads of a logits row, padded
constexpr int kWarps = 8;                  // warps per CTA

// The 16-byte packs of this lane's 8 elements of a row: one for bfloat16, two for float32.
template <typename T> struct RowPack { uint4 v[sizeof(T) == 2 ? 1 : 2]; };

template <typename T>
__device__ __forceinline__ RowPack<T> load_pack(const T* row, int lane) {
  RowPack<T> r;
  r.v[0] = ld_stream(row + lane * kPerLane);
  if constexpr (sizeof(T) == 4) r.v[1] = ld_stream(row + lane * kPerLane + 4);
  return r;
}
template <typename T>
__device__ __forceinline__ void unpack_row(const RowPack<T>& r, float (&f)[kPerLane]) {
  unpack<T>(r.v[0], f);
  if constexpr (sizeof(T) == 4) unpack<T>(r.v[1], f + 4);
}

// Ring slot j holds the latest position congruent to j (mod W) that is below nt, the number of
// tokens seen; the query, at position nt, sees positions nt - W .. nt (torch/modules.py:155-184).
// Once the ring is full every slot holds such a position; before that only slots below nt are
// filled.  So the visible slots are exactly j < nt.
__device__ __forceinline__ int visible_slots(int nt, int W) { return nt < W ? nt : W; }

// The visible entries of a sequence are numbered 0 .. n_vis: ring slots 0 .. n_vis - 1, then the
// new token.  CTA c of kSplits takes entries [c * chunk, (c + 1) * chunk), its warp w every 8th of
// them starting at w.
__device__ __forceinline__ int chunk_of(int total) { return (total + kSplits - 1) / kSplits; }

// grid (B, kSplits).  logits: float [B, W + 1, 16] (head-minor; row e = visible entry e);
// stats: float2 [B, kSplits, kN] = the maximum of the CTA's logits of a head and the sum of
// exp(logit - maximum) over them.
template <typename T, int kN>
__global__ void __launch_bounds__(kWarps * 32)
attn_decode_logits_kernel(const T* __restrict__ q, const T* __restrict__ k_new,
                          const T* __restrict__ keys, const int* __restrict__ num_tokens, int W,
                          float* __restrict__ logits, float2* __restrict__ stats) {
  constexpr bool kBf16 = Traits<T>::kBf16;
  constexpr int kBatch = sizeof(T) == 2 ? 8 : 4;   // rows whose loads are in flight together
  __shared__ float2 s_part[kWarps][kN];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = num_tokens[b];
  const int n_vis = visible_slots(nt, W);
  const int total = n_vis + 1;
  const int chunk = chunk_of(total);
  const int e_begin = blockIdx.y * chunk, e_end = min(e_begin + chunk, total);
  const float scale = 0.0625f;                     // 256^-1/2
  float qf[kN][kPerLane];
#pragma unroll
  for (int n = 0; n < kN; ++n) {
    const RowPack<T> r = load_pack<T>(q + ((int64_t)b * kN + n) * kHdD, lane);
    unpack_row<T>(r, qf[n]);
  }
  float* lg = logits + (int64_t)b * (W + 1) * kHeadPad;
  float m_run = kMasked, l_run = 0.0f;             // lanes < kN: this warp's statistics of head `lane`
  for (int e0 = e_begin + warp; e0 < e_end; e0 += kWarps * kBatch) {
    RowPack<T> raw[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int e = e0 + u * kWarps;
      if (e < e_end)
        raw[u] = load_pack<T>(e == n_vis ? k_new + (int64_t)b * kHdD
                                         : keys + ((int64_t)b * W + e) * kHdD, lane);
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int e = e0 + u * kWarps;
      if (e < e_end) {                             // (the same for every lane of the warp)
        float kf[kPerLane];
        unpack_row<T>(raw[u], kf);
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
          lg[(int64_t)e * kHeadPad + lane] = mine;
          const float m_new = fmaxf(m_run, mine);
          l_run = l_run * __expf(m_run - m_new) + __expf(mine - m_new);
          m_run = m_new;
        }
      }
    }
  }
  if (lane < kN) s_part[warp][lane] = make_float2(m_run, l_run);
  __syncthreads();
  if (threadIdx.x < kN) {
    float m = kMasked, l = 0.0f;
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, s_part[w][threadIdx.x].x);
    for (int w = 0; w < kWarps; ++w) {
      const float2 p = s_part[w][threadIdx.x];
      if (p.x > kMasked) l += p.y * __expf(p.x - m);
    }
    stats[((int64_t)b * kSplits + blockIdx.y) * kN + threadIdx.x] = make_float2(m, l);
  }
}

// grid (B, kSplits): CTA (b, c) multiplies the probabilities of its entries with their value rows,
// all 256 columns (a lane holds 8 of them), for the kN heads.  partial: float [B, kSplits, kN, 256].
template <typename T, int kN>
__global__ void __launch_bounds__(kWarps * 32)
attn_decode_values_kernel(const float* __restrict__ logits, const float2* __restrict__ stats,
                          const T* __restrict__ v_new, const T* __restrict__ values,
                          const int* __restrict__ num_tokens, int W, float* __restrict__ partial) {
  constexpr bool kBf16 = Traits<T>::kBf16;
  constexpr int kBatch = sizeof(T) == 2 ? 8 : 4;
  static_assert(kN <= kHeadPad, "a logits row holds 16 heads");
  __shared__ float s_acc[kWarps / 2][kN][kHdD];    // 40 KiB at 10 heads
  __shared__ float s_stat[2][kHeadPad];            // maximum and 1 / sum of every head
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = num_tokens[b];
  const int n_vis = visible_slots(nt, W);
  const int total = n_vis + 1;
  const int chunk = chunk_of(total);
  const int e_begin = blockIdx.y * chunk, e_end = min(e_begin + chunk, total);
  const float* lg = logits + (int64_t)b * (W + 1) * kHeadPad;
  if (threadIdx.x < kHeadPad) {
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
  const float my_m = s_stat[0][lane & (kHeadPad - 1)], my_inv = s_stat[1][lane & (kHeadPad - 1)];
  float acc[kN][kPerLane];
#pragma unroll
  for (int n = 0; n < kN; ++n)
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) acc[n][i] = 0.0f;
  for (int e0 = e_begin + warp; e0 < e_end; e0 += kWarps * kBatch) {
    RowPack<T> raw[kBatch];
    float lgv[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int e = e0 + u * kWarps;
      lgv[u] = kMasked;
      if (e < e_end) {
        raw[u] = load_pack<T>(e == n_vis ? v_new + (int64_t)b * kHdD
                                         : values + ((int64_t)b * W + e) * kHdD, lane);
        if (lane < kN) lgv[u] = lg[(int64_t)e * kHeadPad + lane];
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int e = e0 + u * kWarps;
      if (e < e_end) {                             // (the same for every lane of the warp)
        float vf[kPerLane];
        unpack_row<T>(raw[u], vf);
        // lane n < kN: the normalised probability of head n, rounded as the reference casts it
        const float p_mine = lgv[u] > kMasked ? rnd<kBf16>(__expf(lgv[u] - my_m) * my_inv) : 0.0f;
#pragma unroll
        for (int n = 0; n < kN; ++n) {
          const float p = __shfl_sync(0xffffffffu, p_mine, n);
#pragma unroll
          for (int i = 0; i < kPerLane; ++i) acc[n][i] = fmaf(p, vf[i], acc[n][i]);
        }
      }
    }
  }
  // the 8 warps: the upper half hands its sums to the lower half, three times over
#pragma unroll
  for (int half = kWarps / 2; half >= 1; half >>= 1) {
    if (warp >= half && warp < 2 * half) {
#pragma unroll
      for (int n = 0; n < kN; ++n)
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) s_acc[warp - half][n][lane * kPerLane + i] = acc[n][i];
    }
    __syncthreads();
    if (warp < half) {
#pragma unroll
      for (int n = 0; n < kN; ++n)
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) acc[n][i] += s_acc[warp][n][lane * kPerLane + i];
    }
    __syncthreads();
  }
  if (warp == 0) {
    float* dst = partial + (((int64_t)b * kSplits + blockIdx.y) * kN) * kHdD + lane * kPerLane;
#pragma unroll
    for (int n = 0; n < kN; ++n) {
      *reinterpret_cast<float4*>(dst + n * kHdD) = make_float4(acc[n][0], acc[n][1], acc[n][2], acc[n][3]);
      *reinterpret_cast<float4*>(dst + n * kHdD + 4) = make_float4(acc[n][4], acc[n][5], acc[n][6], acc[n][7]);
    }
  }
}

// grid (B), 256 threads = the 256 columns: out [B, kN, 256] = the rounded sum of the partials; then
// (update != 0) the new key and value take ring slot num_tokens % W and num_tokens grows by one.
template <typename T, int kN>
__global__ void __launch_bounds__(kHdD)
attn_decode_finish_kernel(const float* __restrict__ partial, const T* __restrict__ k_new,
                          const T* __restrict__ v_new, T* __restrict__ keys, T* __restrict__ values,
                          int* __restrict__ num_tokens, int W, int update, T* __restrict__ out) {
  const int b = blockIdx.x, c = threadIdx.x;
  const int nt = num_tokens[b];
#pragma unroll
  for (int n = 0; n < kN; ++n) {
    float a = 0.0f;
#pragma unroll
    for (int s = 0; s < kSplits; ++s) a += partial[(((int64_t)b * kSplits + s) * kN + n) * kHdD + c];
    out[((int64_t)b * kN + n) * kHdD + c] = static_cast<T>(a);
  }
  if (update) {
    const int slot = nt % W;
    keys[((int64_t)b * W + slot) * kHdD + c] = k_new[(int64_t)b * kHdD + c];
    values[((int64_t)b * W + slot) * kHdD + c] = v_new[(int64_t)b * kHdD + c];
    __syncthreads();                                // every thread has read nt
    if (c == 0) num_tokens[b] = nt + 1;
  }
}

// the logits [B, W + 1, 16], the per-CTA softmax statistics [B, kSplits, N], the partial sums
// [B, kSplits, N, 256]
size_t logits_bytes(int64_t B, int W) {
  return (((size_t)B * (W + 1) * kHeadPad * sizeof(float)) + 255) & ~(size_t)255;
}
size_t stats_bytes(int64_t B, int N) {
  return (((size_t)B * kSplits * N * sizeof(float2)) + 255) & ~(size_t)255;
}
size_t partial_bytes(int64_t B, int N) {
  return (((size_t)B * kSplits * N * kHdD * sizeof(float)) + 255) & ~(size_t)255;
}

template <typename T, int kN>
cudaError_t launch_decode_t(const void* q, const void* k_new, const void* v_new, void* keys,
                            void* values, int* num_tokens, int64_t B, int W, int update, void* out,
                            void* ws, cudaStream_t s) {
  uint8_t* base = reinterpret_cast<uint8_t*>(ws);
  float* lg = reinterpret_cast<float*>(base);
  float2* st = reinterpret_cast<float2*>(base + logits_bytes(B, W));
  float* part = reinterpret_cast<float*>(base + logits_bytes(B, W) + stats_bytes(B, kN));
  attn_decode_logits_kernel<T, kN><<<dim3((unsigned)B, kSplits), kWarps * 32, 0, s>>>(
      (const T*)q, (const T*)k_new, (const T*)keys, num_tokens, W, lg, st);
  attn_decode_values_kernel<T, kN><<<dim3((unsigned)B, kSplits), kWarps * 32, 0, s>>>(
      lg, st, (const T*)v_new, (const T*)values, num_tokens, W, part);
  attn_decode_finish_kernel<T, kN><<<(unsigned)B, kHdD, 0, s>>>(
      part, (const T*)k_new, (const T*)v_new, (T*)keys, (T*)values, num_tokens, W, update, (T*)out);
  return cudaGetLastError();
}

}  // namespace

bool attention_decode_supported(int hd, int N, int W) {
  const bool heads = N == 1 || N == 2 || N == 4 || N == 8 || N == 10;
  return hd == kHdD && heads && W >= 1;
}

size_t attention_decode_workspace_bytes(int64_t B, int N, int W) {
  return logits_bytes(B, W) + stats_bytes(B, N) + partial_bytes(B, N);
}

cudaError_t launch_attention_decode(const void* q, const void* k_new, const void* v_new, void* keys,
                                    void* values, int* num_tokens, int64_t B, int N, int W,
                                    int dtype, int update, void* out, void* ws, cudaStream_t s) {
  if (B == 0) return cudaSuccess;
#define RGK_DEC(NN)                                                                              \
  case NN:                                                                                       \
    return dtype == 1 ? launch_decode_t<__nv_bfloat16, NN>(q, k_new, v_new, keys, values,        \
                                                           num_tokens, B, W, update, out, ws, s) \
                      : launch_decode_t<float, NN>(q, k_new, v_new, keys, values, num_tokens, B, \
                                                   W, update, out, ws, s)
  switch (N) {
    RGK_DEC(1); RGK_DEC(2); RGK_DEC(4); RGK_DEC(8); RGK_DEC(10);
    default: return cudaErrorInvalidValue;
  }
#undef RGK_DEC
}

}  // namespace rgk
