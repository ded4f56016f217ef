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
// All three are bandwidth work on the ring (2 W 256 elements per sequence): 16 CTAs per sequence,
// every warp with the loads of a whole batch of rows in flight before it uses the first.  The
// float32 kernels do their arithmetic on the CUDA cores (a warp reads a 256-element row as one pack
// per lane; ~200 instructions per row, which is what bounds them); the bfloat16 kernels use the
// warp-level tensor-core instruction (m16n8k16), ~6 instructions per row - a tile is 16 ring rows
// by 16 padded heads, far below the 128-row tiles of tcgen05.
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

// ------------------------------------------------------------------------------------------------
// bfloat16: the same two kernels on the warp-level tensor-core instruction (m16n8k16), which cuts
// the instruction count per ring row from ~200 to ~6 and leaves the kernels to the memory system.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two running (maximum, sum of exponentials) pairs into one.
__device__ __forceinline__ void merge_stats(float& m, float& l, float mo, float lo) {
  const float m_new = fmaxf(m, mo);
  l = l * __expf(m - m_new) + lo * __expf(mo - m_new);
  m = m_new;
}

// Logits of a tile of 16 entries x 16 (padded) heads per warp.  In the fragments of the
// instruction, lane (g = lane / 4, t = lane % 4) holds rows g and g + 8 of A and column g of B at
// the contraction indices 2t, 2t+1, 2t+8, 2t+9.  The contraction runs over the 256 elements of a
// row in any order, as long as A and B agree on it: a lane therefore takes the 8 consecutive
// elements 32 i + 8 t .. + 7 of its rows with one 16-byte load and feeds them to two instructions
// (elements 0-3, then 4-7), and does the same with its head's row of q.
template <int kN>
__global__ void __launch_bounds__(kWarps * 32)
attn_decode_logits_mma_kernel(const __nv_bfloat16* __restrict__ q,
                              const __nv_bfloat16* __restrict__ k_new,
                              const __nv_bfloat16* __restrict__ keys,
                              const int* __restrict__ num_tokens, int W,
                              float* __restrict__ logits, float2* __restrict__ stats) {
  constexpr int kTiles = kN > 8 ? 2 : 1;           // groups of 8 heads
  __shared__ float2 s_part[kWarps][kHeadPad];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int nt = num_tokens[b];
  const int n_vis = visible_slots(nt, W);
  const int total = n_vis + 1;
  const int chunk = chunk_of(total);
  const int e_begin = blockIdx.y * chunk, e_end = min(e_begin + chunk, total);
  uint4 qb[kTiles][8];
#pragma unroll
  for (int h = 0; h < kTiles; ++h) {
    const int head = h * 8 + g;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      qb[h][i] = head < kN ? *reinterpret_cast<const uint4*>(q + ((int64_t)b * kN + head) * kHdD + i * 32 + t * 8)
                           : make_uint4(0u, 0u, 0u, 0u);
  }
  float* lg = logits + (int64_t)b * (W + 1) * kHeadPad;
  float m_run[kTiles][2], l_run[kTiles][2];        // heads 8 h + 2 t and + 1, over this lane's rows
#pragma unroll
  for (int h = 0; h < kTiles; ++h) {
    m_run[h][0] = m_run[h][1] = kMasked;
    l_run[h][0] = l_run[h][1] = 0.0f;
  }
  for (int e0 = e_begin + 16 * warp; e0 < e_end; e0 += 16 * kWarps) {
    const int r0 = e0 + g, r1 = e0 + g + 8;
    // rows past the end of the CTA's range are loaded as its last row and ignored
    const int c0 = min(r0, e_end - 1), c1 = min(r1, e_end - 1);
    const __nv_bfloat16* p0 = (c0 == n_vis ? k_new + (int64_t)b * kHdD : keys + ((int64_t)b * W + c0) * kHdD) + t * 8;
    const __nv_bfloat16* p1 = (c1 == n_vis ? k_new + (int64_t)b * kHdD : keys + ((int64_t)b * W + c1) * kHdD) + t * 8;
    uint4 ra[8], rb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ra[i] = ld_stream(p0 + i * 32);
      rb[i] = ld_stream(p1 + i * 32);
    }
    float acc[kTiles][4];
#pragma unroll
    for (int h = 0; h < kTiles; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int h = 0; h < kTiles; ++h) {
        mma_16816(acc[h], ra[i].x, rb[i].x, ra[i].y, rb[i].y, qb[h][i].x, qb[h][i].y);
        mma_16816(acc[h], ra[i].z, rb[i].z, ra[i].w, rb[i].w, qb[h][i].z, qb[h][i].w);
      }
    }
    // two tensor operations in the reference: the contraction, then the scaling by 256^-1/2
#pragma unroll
    for (int h = 0; h < kTiles; ++h) {
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[h][j] = round_bf16(round_bf16(acc[h][j]) * 0.0625f);
      if (r0 < e_end) {
        *reinterpret_cast<float2*>(lg + (int64_t)r0 * kHeadPad + h * 8 + t * 2) = make_float2(acc[h][0], acc[h][1]);
        merge_stats(m_run[h][0], l_run[h][0], acc[h][0], 1.0f);
        merge_stats(m_run[h][1], l_run[h][1], acc[h][1], 1.0f);
      }
      if (r1 < e_end) {
        *reinterpret_cast<float2*>(lg + (int64_t)r1 * kHeadPad + h * 8 + t * 2) = make_float2(acc[h][2], acc[h][3]);
        merge_stats(m_run[h][0], l_run[h][0], acc[h][2], 1.0f);
        merge_stats(m_run[h][1], l_run[h][1], acc[h][3], 1.0f);
      }
    }
  }
  // the 8 lanes that share t, then the warps
#pragma unroll
  for (int h = 0; h < kTiles; ++h)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m_run[h][j], o);
        const float lo = __shfl_xor_sync(0xffffffffu, l_run[h][j], o);
        merge_stats(m_run[h][j], l_run[h][j], mo, lo);
      }
      if (g == 0) s_part[warp][h * 8 + t * 2 + j] = make_float2(m_run[h][j], l_run[h][j]);
    }
  __syncthreads();
  if (threadIdx.x < kN) {
    float m = kMasked, l = 0.0f;
    for (int w = 0; w < kWarps; ++w) {
      const float2 p = s_part[w][threadIdx.x];
      merge_stats(m, l, p.x, p.y);
    }
    stats[((int64_t)b * kSplits + blockIdx.y) * kN + threadIdx.x] = make_float2(m, l);
  }
}

// Probabilities x values on the same instruction.  All warps of a CTA walk the CTA's entries, 16
// at a time, each for its own 32 of the 256 columns, so no sums cross warps: A = the rounded
// probabilities [16 padded heads x 16 entries], formed in registers from the logits (every warp
// repeats that small step), B = 16 entries x 32 columns of the values, which have to be read
// across rows (two entries of one column per register): the warp copies the piece into shared
// memory with 16-byte loads and takes the fragments back with ldmatrix.trans.  Rows of the piece
// are padded to 80 bytes so that the 8 row addresses of a matrix fall into different banks.
constexpr int kPieceRow = 64 + 16;
constexpr int kPiece = 16 * kPieceRow;                           // 1280 bytes per warp
constexpr int kAhead = 5;                                        // tiles whose loads are in flight

template <int kN>
__global__ void __launch_bounds__(kWarps * 32)
attn_decode_values_mma_kernel(const float* __restrict__ logits, const float2* __restrict__ stats,
                              const __nv_bfloat16* __restrict__ v_new,
                              const __nv_bfloat16* __restrict__ values,
                              const int* __restrict__ num_tokens, int W,
                              float* __restrict__ partial) {
  constexpr int kTiles = kN > 8 ? 2 : 1;           // groups of 8 heads (rows g and g + 8 of A)
  __shared__ __align__(16) uint8_t s_piece[kWarps][kPiece];
  __shared__ float s_stat[2][kHeadPad];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int nt = num_tokens[b];
  const int n_vis = visible_slots(nt, W);
  const int total = n_vis + 1;
  const int chunk = chunk_of(total);
  const int e_begin = blockIdx.y * chunk, e_end = min(e_begin + chunk, total);
  const float* lg = logits + (int64_t)b * (W + 1) * kHeadPad;
  {
    // thread (head, CTA of the logits kernel) takes one pair of statistics; the 16 lanes of a head
    // merge theirs in four steps
    static_assert(kSplits == 16 && kWarps * 32 == kHeadPad * kSplits, "one thread per pair");
    const int head = threadIdx.x >> 4, c = threadIdx.x & 15;
    float m = kMasked, l = 0.0f;
    if (head < kN) {
      const float2 p = stats[((int64_t)b * kSplits + c) * kN + head];
      m = p.x;
      l = p.y;
    }
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m, o), lo = __shfl_xor_sync(0xffffffffu, l, o);
      merge_stats(m, l, mo, lo);
    }
    if (c == 0) {
      s_stat[0][head] = m;
      s_stat[1][head] = l > 0.0f ? 1.0f / l : 0.0f;
    }
  }
  __syncthreads();
  // this lane's two heads (rows g and g + 8 of A)
  const float m0 = s_stat[0][g], i0 = s_stat[1][g], m1 = s_stat[0][g + 8], i1 = s_stat[1][g + 8];
  uint8_t* piece = s_piece[warp];
  const uint32_t piece_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(piece));
  // ldmatrix.x4.trans: lane L gives the address of row L % 8 of matrix L / 8; matrices 0 and 1 are
  // entries 0-7 and 8-15 of one group of 8 columns, matrices 2 and 3 the same of the next group
  const uint32_t ld_base = piece_u32 + (((lane >> 3) & 1) * 8 + (lane & 7)) * kPieceRow + (lane >> 4) * 16;
  // a lane copies 16 bytes of rows lane / 4 and lane / 4 + 8 of a tile: columns 32 warp + 8 t .. + 7
  const int col = warp * 32 + t * 8;
  auto row_ptr = [&](int e) {
    return (e == n_vis ? v_new + (int64_t)b * kHdD : values + ((int64_t)b * W + e) * kHdD) + col;
  };
  // the logit of entry e and head `head`, or "none"
  auto logit = [&](int e, int head) {
    return (e < e_end && head < kN) ? lg[(int64_t)e * kHeadPad + head] : kMasked;
  };
  auto prob = [&](float v, float m, float inv) {
    return v > kMasked ? round_bf16(__expf(v - m) * inv) : 0.0f;
  };
  float acc[4][4];                                 // four groups of 8 columns
#pragma unroll
  for (int n = 0; n < 4; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
  for (int e0 = e_begin; e0 < e_end; e0 += 16 * kAhead) {
    uint4 lo[kAhead], hi[kAhead];                  // rows past the end as zeros
    float lv[kAhead][kTiles][4];                   // this lane's logits: entries 2t, 2t+1, 2t+8, 2t+9
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int ea = e0 + 16 * u + g, eb = ea + 8;
      lo[u] = ea < e_end ? ld_stream(row_ptr(ea)) : make_uint4(0u, 0u, 0u, 0u);
      hi[u] = eb < e_end ? ld_stream(row_ptr(eb)) : make_uint4(0u, 0u, 0u, 0u);
      const int pa = e0 + 16 * u + 2 * t;
#pragma unroll
      for (int h = 0; h < kTiles; ++h) {
        lv[u][h][0] = logit(pa, g + 8 * h);
        lv[u][h][1] = logit(pa + 1, g + 8 * h);
        lv[u][h][2] = logit(pa + 8, g + 8 * h);
        lv[u][h][3] = logit(pa + 9, g + 8 * h);
      }
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int et = e0 + 16 * u;
      if (et < e_end) {                            // (the same for every lane of the warp)
        // the probabilities of this lane's heads at its four pairs of entries
        const uint32_t a0 = pack_bf16x2(prob(lv[u][0][0], m0, i0), prob(lv[u][0][1], m0, i0));
        const uint32_t a2 = pack_bf16x2(prob(lv[u][0][2], m0, i0), prob(lv[u][0][3], m0, i0));
        uint32_t a1 = 0u, a3 = 0u;
        if (kTiles == 2) {
          a1 = pack_bf16x2(prob(lv[u][kTiles - 1][0], m1, i1), prob(lv[u][kTiles - 1][1], m1, i1));
          a3 = pack_bf16x2(prob(lv[u][kTiles - 1][2], m1, i1), prob(lv[u][kTiles - 1][3], m1, i1));
        }
        __syncwarp();                              // the previous tile's fragments have been read
        *reinterpret_cast<uint4*>(piece + g * kPieceRow + t * 16) = lo[u];
        *reinterpret_cast<uint4*>(piece + (g + 8) * kPieceRow + t * 16) = hi[u];
        __syncwarp();
#pragma unroll
        for (int n2 = 0; n2 < 2; ++n2) {           // two groups of 8 columns per ldmatrix
          uint32_t b0, b1, b2, b3;
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(ld_base + n2 * 32));
          mma_16816(acc[2 * n2], a0, a1, a2, a3, b0, b1);
          mma_16816(acc[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
  }
  // C fragment: (head g, columns 8 n + 2 t, + 1) and (head g + 8, the same columns)
  float* dst = partial + (((int64_t)b * kSplits + blockIdx.y) * kN) * kHdD + warp * 32 + t * 2;
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    if (g < kN) *reinterpret_cast<float2*>(dst + g * kHdD + n * 8) = make_float2(acc[n][0], acc[n][1]);
    if (g + 8 < kN) *reinterpret_cast<float2*>(dst + (g + 8) * kHdD + n * 8) = make_float2(acc[n][2], acc[n][3]);
  }
}

// grid (B, kN), 256 threads = the 256 columns: out [B, kN, 256] = the rounded sum of the partials;
// then (update != 0; the CTAs of head 0) the new key and value take ring slot num_tokens % W and
// num_tokens grows by one.
template <typename T, int kN>
__global__ void __launch_bounds__(kHdD)
attn_decode_finish_kernel(const float* __restrict__ partial, const T* __restrict__ k_new,
                          const T* __restrict__ v_new, T* __restrict__ keys, T* __restrict__ values,
                          int* __restrict__ num_tokens, int W, int update, T* __restrict__ out) {
  const int b = blockIdx.x, n = blockIdx.y, c = threadIdx.x;
  float a = 0.0f;
#pragma unroll
  for (int s = 0; s < kSplits; ++s) a += partial[(((int64_t)b * kSplits + s) * kN + n) * kHdD + c];
  out[((int64_t)b * kN + n) * kHdD + c] = static_cast<T>(a);
  if (update && n == 0) {
    const int nt = num_tokens[b];
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
  const dim3 grid((unsigned)B, kSplits);
  if constexpr (Traits<T>::kBf16) {
    attn_decode_logits_mma_kernel<kN><<<grid, kWarps * 32, 0, s>>>(
        (const T*)q, (const T*)k_new, (const T*)keys, num_tokens, W, lg, st);
    attn_decode_values_mma_kernel<kN><<<grid, kWarps * 32, 0, s>>>(
        lg, st, (const T*)v_new, (const T*)values, num_tokens, W, part);
  } else {
    attn_decode_logits_kernel<T, kN><<<grid, kWarps * 32, 0, s>>>(
        (const T*)q, (const T*)k_new, (const T*)keys, num_tokens, W, lg, st);
    attn_decode_values_kernel<T, kN><<<grid, kWarps * 32, 0, s>>>(
        lg, st, (const T*)v_new, (const T*)values, num_tokens, W, part);
  }
  attn_decode_finish_kernel<T, kN><<<dim3((unsigned)B, kN), kHdD, 0, s>>>(
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
