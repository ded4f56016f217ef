// Local (sliding-window) multi-query attention of the attention residual blocks, prefill form
// (recurrentgemma torch/modules.py:399-493 with the helpers at 58-140), bfloat16, head dimension
// 256, one key/value head:
//   rope_kernel         rotary embedding of queries and keys (torch/modules.py:58-86);
//   attn_bounds_kernel  per token the first visible key: max(start of its document, t - window)
//                       (the mask of torch/modules.py:89-140 is "lo(t) <= s <= t": documents are
//                       contiguous, so "same segment" is "not before the start of mine");
//   transpose_v_kernel  values [B,T,256] -> [B,256,Tp], key index contiguous, zero padded: the
//                       second contraction then has a K-major B operand like the first;
//   attn_prefill_kernel the attention itself on tcgen05.
//
// The reference rounds the logits to bfloat16, takes the softmax of the masked logits in float32
// over the WHOLE row and casts the normalised probabilities to bfloat16 before the second
// contraction.  To round what the reference rounds, the kernel makes two passes over the key tiles
// of a query tile: pass 1 computes every row's maximum and sum (online), pass 2 recomputes the
// logits, forms the normalised probabilities, rounds them, and accumulates P V on the tensor cores.
//
// A unit of work is (sequence, query head, 128 queries); units are dealt out round-robin to
// persistent CTAs.  Roles in a CTA (10 warps):
//   warps 0-7  softmax: group g = warp / 4 takes the key tiles of parity g (its own S accumulator
//              and P buffer), thread = query row (TMEM lane quarter warp % 4);
//   warp 8     TMA producer: per key tile four K-slices of 64 of the query tile and of the key tile
//              into a 3-stage ring, in pass 2 also the two 64-key slices of the transposed values;
//   warp 9     TMEM allocation and MMA issue: S = Q K^T (M 128, N 128, 16 K-steps) into S[parity],
//              O += P V (M 128, N 256, 8 K-steps) once the group has written P[parity].
// TMEM: S[0], S[1] (128 columns each), O (256 columns).  All waits are bounded; on expiry the
// status word is raised and the CTA runs to its end.
#include <cuda.h>
#include <math.h>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tc_common.cuh"

namespace rgk {
namespace {

// ------------------------------------------------------------------------------------------------
// Rotary embedding: x [rows, heads, hd] in place, positions [rows].  The first half of a head is
// rotated in pairs (i, i + hd/4), the second half is left alone.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, const void* __restrict__ pos, int pos64, int64_t rows,
                            int heads, int hd) {
  constexpr bool kBf16 = Traits<T>::kBf16;
  const int quarter = hd / 4;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = rows * heads * quarter;
  if (idx >= total) return;
  const int i = (int)(idx % quarter);
  const int64_t rh = idx / quarter;            // row * heads + head
  const int64_t row = rh / heads;
  const float p = pos64 ? (float)reinterpret_cast<const long long*>(pos)[row]
                        : (float)reinterpret_cast<const int*>(pos)[row];
  const float exponent = 2.0f * (float)i / (float)(hd / 2);
  const float inv = 1.0f / powf(10000.0f, exponent);
  const float ang = p * inv;
  const float sn = rnd<kBf16>(sinf(ang)), cs = rnd<kBf16>(cosf(ang));
  T* h = x + rh * hd;
  const float a = (float)h[i], b = (float)h[i + quarter];
  const float o0 = rnd<kBf16>(rnd<kBf16>(a * cs) - rnd<kBf16>(b * sn));
  const float o1 = rnd<kBf16>(rnd<kBf16>(b * cs) + rnd<kBf16>(a * sn));
  h[i] = (T)o0;
  h[i + quarter] = (T)o1;
}

// lo[b, t] = max(start of the document of token t, t - window); one warp per sequence.
__global__ void attn_bounds_kernel(const void* __restrict__ pos, int pos64, int B, int T_, int window,
                                   int* __restrict__ lo) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  int start = 0;                                // tokens before the first document start: segment 0
  for (int t0 = 0; t0 < T_; t0 += 32) {
    const int t = t0 + lane;
    const bool z = t < T_ && pos_is_zero(pos, pos64, (int64_t)b * T_ + t);
    const unsigned m = __ballot_sync(0xffffffffu, z);
    const unsigned upto = m & (lane == 31 ? 0xffffffffu : ((2u << lane) - 1u));
    const int mine = upto ? t0 + 31 - __clz(upto) : start;
    if (t < T_) lo[(int64_t)b * T_ + t] = max(mine, t - window);
    if (m) start = t0 + 31 - __clz(m);
  }
}

// v [B, T, 256] -> vt [B, 256, Tp]; columns T .. Tp-1 are zero.
__global__ void transpose_v_kernel(const __nv_bfloat16* __restrict__ v, int T_, int Tp,
                                   __nv_bfloat16* __restrict__ vt) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int b = blockIdx.z, t0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += 8) {
    const int t = t0 + r;
    tile[r][threadIdx.x] = t < T_ ? v[((int64_t)b * T_ + t) * 256 + d0 + threadIdx.x] : __float2bfloat16(0.0f);
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += 8) {
    const int t = t0 + threadIdx.x;
    if (t < Tp) vt[((int64_t)b * 256 + d0 + r) * Tp + t] = tile[threadIdx.x][r];
  }
}

// ------------------------------------------------------------------------------------------------
// The attention kernel.
// ------------------------------------------------------------------------------------------------
constexpr int kHd = 256;                  // head dimension = K of Q K^T, N of P V
constexpr int kTq = 128, kTk = 128;       // queries / keys per tile
constexpr int kSl = 64;                   // slice width (one 128-byte swizzle row of bfloat16)
constexpr int kQkStage = 2 * kTq * kSl * 2;          // Q slice + K slice: 32 KiB
constexpr int kRingA = 3;
constexpr int kVStage = kHd * kSl * 2;               // a 64-key slice of V^T: 32 KiB
constexpr int kPBytes = kTq * kTk * 2;               // 32 KiB per group
constexpr int kOffQk = 0;
constexpr int kOffV = kRingA * kQkStage;             //  98304
constexpr int kOffP = kOffV + 2 * kVStage;           // 163840
// The groups' partial (max, sum) of a row, float2 [2 groups][128 rows], are exchanged between the
// passes through the first bytes of the P buffers: no MMA reads P then (the logits of this unit's
// pass 1 were produced after the last P V of the previous unit, and tcgen05 runs in issue order).
constexpr int kOffMl = kOffP;
constexpr int kOffBarA = kOffP + 2 * kPBytes;        // 229376
constexpr int kNumBarA = 2 * kRingA + 4 + 8 + 2;     // ring, v, s_full/s_empty/p_full/p_empty [2], o
constexpr int kOffTmemA = kOffBarA + kNumBarA * 8;
constexpr int kOffAbortA = kOffTmemA + 4;
constexpr int kSmemA = kOffAbortA + 4 + 1024;
static_assert(kSmemA <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");
constexpr int kSoftWarps = 8;
constexpr int kThreadsA = (kSoftWarps + 2) * 32;
constexpr uint32_t kIdescS = tc_idesc_bf16(kTq, kTk);
constexpr uint32_t kIdescO = tc_idesc_bf16(kTq, kHd);
constexpr float kNegBig = -3.0e38f;

__global__ void __launch_bounds__(kThreadsA, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_vt, const int* __restrict__ lo_all, int B,
                    int T_, int N, int window, int n_units, __nv_bfloat16* __restrict__ out,
                    int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar0 = s_base + kOffBarA;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kRingA + s); };
  auto bar_v_full = [&](int s) { return bar0 + 8u * (2 * kRingA + s); };
  auto bar_v_empty = [&](int s) { return bar0 + 8u * (2 * kRingA + 2 + s); };
  auto bar_s_full = [&](int g) { return bar0 + 8u * (2 * kRingA + 4 + g); };
  auto bar_s_empty = [&](int g) { return bar0 + 8u * (2 * kRingA + 6 + g); };
  auto bar_p_full = [&](int g) { return bar0 + 8u * (2 * kRingA + 8 + g); };
  auto bar_p_empty = [&](int g) { return bar0 + 8u * (2 * kRingA + 10 + g); };
  const uint32_t bar_o_full = bar0 + 8u * (2 * kRingA + 12);
  const uint32_t bar_o_empty = bar0 + 8u * (2 * kRingA + 13);
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + kOffTmemA);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffAbortA);
  float2* s_ml = reinterpret_cast<float2*>(smem + kOffMl);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (T_ + kTq - 1) / kTq;
  const int n_my = (n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int s = 0; s < kRingA; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_v_full(s), 1); mbar_init(bar_v_empty(s), 1);
      mbar_init(bar_s_full(s), 1); mbar_init(bar_s_empty(s), 4);
      mbar_init(bar_p_full(s), 4); mbar_init(bar_p_empty(s), 1);
    }
    mbar_init(bar_o_full, 1);
    mbar_init(bar_o_empty, 4);
    mbar_fence_init();
  }
  if (warp == kSoftWarps + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(s_base + kOffTmemA), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  // unit -> (sequence, head, query tile); the key tiles it needs
  auto unit_of = [&](int i, int& b, int& n, int& t0, int& j_lo, int& j_hi) {
    const int u = blockIdx.x + i * gridDim.x;
    const int qt = u % q_tiles, bn = u / q_tiles;
    n = bn % N;
    b = bn / N;
    t0 = qt * kTq;
    j_lo = max(0, t0 - window) / kTk;
    j_hi = min(t0 + kTq - 1, T_ - 1) / kTk;       // inclusive
  };

  if (warp == kSoftWarps) {
    // ------------------------------ TMA producer --------------------------------------------------
    if (lane == 0) {
      unsigned it = 0, iv = 0;
      bool ok = true;
      for (int i = 0; i < n_my && ok; ++i) {
        int b, n, t0, j_lo, j_hi;
        unit_of(i, b, n, t0, j_lo, j_hi);
        for (int pass = 0; pass < 2 && ok; ++pass) {
          for (int j = j_lo; j <= j_hi && ok; ++j) {
            for (int ks = 0; ks < kHd / kSl; ++ks, ++it) {
              const int s = it % kRingA;
              ok = mbar_wait(bar_empty(s), ((it / kRingA) & 1) ^ 1, s_abort);
              if (!ok) break;
              mbar_expect_tx(bar_full(s), kQkStage);
              const uint32_t dst = s_base + kOffQk + s * kQkStage;
              tma_load_3d(dst, &map_q, n * kHd + ks * kSl, t0, b, bar_full(s));
              tma_load_3d(dst + kTq * kSl * 2, &map_k, ks * kSl, j * kTk, b, bar_full(s));
            }
            if (pass == 1 && ok) {
              for (int c = 0; c < kTk / kSl; ++c, ++iv) {
                const int s = iv & 1;
                ok = mbar_wait(bar_v_empty(s), ((iv >> 1) & 1) ^ 1, s_abort);
                if (!ok) break;
                mbar_expect_tx(bar_v_full(s), kVStage);
                tma_load_3d(s_base + kOffV + s * kVStage, &map_vt, j * kTk + c * kSl, 0, b,
                            bar_v_full(s));
              }
            }
          }
        }
      }
    }
  } else if (warp == kSoftWarps + 1) {
    // ------------------------------ MMA issue -----------------------------------------------------
    if (lane == 0) {
      unsigned it = 0, iv = 0;
      unsigned s_use[2] = {0, 0}, p_use[2] = {0, 0};
      bool ok = true;
      auto issue_qk = [&](int g) {
        // S[g] = Q K^T for the next key tile in the ring
        if (ok) ok = mbar_wait(bar_s_empty(g), (s_use[g] & 1) ^ 1, s_abort);
        ++s_use[g];
        if (ok) tc_fence_after();
        for (int ks = 0; ks < kHd / kSl && ok; ++ks, ++it) {
          const int s = it % kRingA;
          ok = mbar_wait(bar_full(s), (it / kRingA) & 1, s_abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t q0 = s_base + kOffQk + s * kQkStage, k0 = q0 + kTq * kSl * 2;
#pragma unroll
          for (int kk = 0; kk < kSl / 16; ++kk)
            tc_mma_bf16(tmem_base + g * kTk, smem_desc_sw128(q0 + kk * 32), smem_desc_sw128(k0 + kk * 32),
                        kIdescS, (ks | kk) != 0 ? 1u : 0u);
          tc_commit(bar_empty(s));
        }
        if (ok) tc_commit(bar_s_full(g));
      };
      auto issue_pv = [&](int g, bool first) {
        // O += P[g] V for the key tile whose probabilities group g has just written
        if (ok) ok = mbar_wait(bar_p_full(g), p_use[g] & 1, s_abort);
        ++p_use[g];
        if (ok) tc_fence_after();
        for (int c = 0; c < kTk / kSl && ok; ++c, ++iv) {
          const int s = iv & 1;
          ok = mbar_wait(bar_v_full(s), (iv >> 1) & 1, s_abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t p0 = s_base + kOffP + g * kPBytes + c * (kTq * kSl * 2);
          const uint32_t v0 = s_base + kOffV + s * kVStage;
#pragma unroll
          for (int kk = 0; kk < kSl / 16; ++kk)
            tc_mma_bf16(tmem_base + 2 * kTk, smem_desc_sw128(p0 + kk * 32), smem_desc_sw128(v0 + kk * 32),
                        kIdescO, (first && c == 0 && kk == 0) ? 0u : 1u);
          tc_commit(bar_v_empty(s));
        }
        if (ok) tc_commit(bar_p_empty(g));
      };
      for (int i = 0; i < n_my && ok; ++i) {
        int b, n, t0, j_lo, j_hi;
        unit_of(i, b, n, t0, j_lo, j_hi);
        const int nt = j_hi - j_lo + 1;
        // pass 1: logits only
        for (int j = 0; j < nt && ok; ++j) issue_qk(j & 1);
        // pass 2: logits one tile ahead of the probabilities
        if (ok) ok = mbar_wait(bar_o_empty, (i & 1) ^ 1, s_abort);
        if (ok) tc_fence_after();
        if (nt > 0) issue_qk(0);
        for (int j = 0; j < nt && ok; ++j) {
          if (j + 1 < nt) issue_qk((j + 1) & 1);
          issue_pv(j & 1, j == 0);
        }
        if (ok) tc_commit(bar_o_full);
      }
    }
  } else {
    // ------------------------------ softmax and epilogue ------------------------------------------
    const int g = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;                     // query row inside the tile = TMEM lane
    const uint32_t t_s = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + g * kTk;
    const uint32_t t_o = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + 2 * kTk;
    uint8_t* p_buf = smem + kOffP + g * kPBytes;
    constexpr float kScale = 0.0625f * 1.4426950408889634f;  // hd^-1/2 log2(e): exponent per logit unit
    unsigned cs = 0, cp = 0;
    bool ok = true;
    for (int i = 0; i < n_my; ++i) {
      int b, n, t0, j_lo, j_hi;
      unit_of(i, b, n, t0, j_lo, j_hi);
      const int nt = j_hi - j_lo + 1;
      const int t = t0 + row;
      const bool row_ok = t < T_;
      // visible keys of this row: lo .. t (a row past the end sees key 0 only; it is never stored)
      const int lo = row_ok ? lo_all[(int64_t)b * T_ + t] : 0;
      const int hi = row_ok ? t : 0;

      // ---- pass 1: row maximum and sum over this group's key tiles --------------------------------
      float m = kNegBig, l = 0.0f;
      for (int j = g; j < nt; j += 2) {
        if (ok) ok = mbar_wait(bar_s_full(g), cs & 1, s_abort);
        ++cs;
        tc_fence_after();
        const int s0 = (j_lo + j) * kTk;
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t acc[32];
          if (ok) {
            tc_ld_32x32(t_s + cc * 32, acc);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) acc[c] = 0u;
          }
          const int sc = s0 + cc * 32;
          float v[32];
          float cm = kNegBig;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float sv = round_bf16(__uint_as_float(acc[c]));
            v[c] = (sc + c >= lo && sc + c <= hi) ? sv : kNegBig;
            cm = fmaxf(cm, v[c]);
          }
          if (cm > kNegBig) {
            const float m_new = fmaxf(m, cm);
            float add = 0.0f;
#pragma unroll
            for (int c = 0; c < 32; ++c) add += v[c] > kNegBig ? ex2f((v[c] - m_new) * kScale) : 0.0f;
            l = l * ex2f((m - m_new) * kScale) + add;
            m = m_new;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(bar_s_empty(g));
      }
      // both groups' partial (m, l) -> the row's final ones
      s_ml[g * kTq + row] = make_float2(m, l);
      named_bar_sync(1, kSoftWarps * 32);
      {
        const float2 o = s_ml[(g ^ 1) * kTq + row];
        const float m_all = fmaxf(m, o.x);
        float l_all = 0.0f;
        if (m > kNegBig) l_all += l * ex2f((m - m_all) * kScale);
        if (o.x > kNegBig) l_all += o.y * ex2f((o.x - m_all) * kScale);
        m = m_all;
        l = l_all;
      }
      named_bar_sync(1, kSoftWarps * 32);      // s_ml may be rewritten by the next unit
      const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;

      // ---- pass 2: normalised probabilities, rounded, into P[g] -----------------------------------
      for (int j = g; j < nt; j += 2) {
        if (ok) ok = mbar_wait(bar_s_full(g), cs & 1, s_abort);
        ++cs;
        if (ok) ok = mbar_wait(bar_p_empty(g), (cp & 1) ^ 1, s_abort);
        ++cp;
        tc_fence_after();
        const int s0 = (j_lo + j) * kTk;
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t acc[32];
          if (ok) {
            tc_ld_32x32(t_s + cc * 32, acc);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) acc[c] = 0u;
          }
          const int sc = s0 + cc * 32;
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float p0 = 0.0f, p1 = 0.0f;
            if (sc + c >= lo && sc + c <= hi)
              p0 = ex2f((round_bf16(__uint_as_float(acc[c])) - m) * kScale) * inv_l;
            if (sc + c + 1 >= lo && sc + c + 1 <= hi)
              p1 = ex2f((round_bf16(__uint_as_float(acc[c + 1])) - m) * kScale) * inv_l;
            pk[c >> 1] = pack_bf16x2(p0, p1);
          }
          // 32 keys = 64 bytes = four 16-byte units of this row in slice cc / 2
          uint8_t* prow = p_buf + (cc >> 1) * (kTq * kSl * 2) + row * 128;
#pragma unroll
          for (int u4 = 0; u4 < 4; ++u4) {
            const int unit = (cc & 1) * 4 + u4;
            *reinterpret_cast<uint4*>(prow + ((unit ^ (row & 7)) << 4)) =
                make_uint4(pk[4 * u4], pk[4 * u4 + 1], pk[4 * u4 + 2], pk[4 * u4 + 3]);
          }
        }
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && ok) {
          mbar_arrive(bar_s_empty(g));
          mbar_arrive(bar_p_full(g));
        }
      }

      // ---- epilogue (group 0): O -> bfloat16 -> encoded [B, T, N * 256] ---------------------------
      if (g == 0) {
        if (ok) ok = mbar_wait(bar_o_full, i & 1, s_abort);
        tc_fence_after();
        __nv_bfloat16* orow = out + ((int64_t)b * T_ + t) * ((int64_t)N * kHd) + (int64_t)n * kHd;
#pragma unroll 1
        for (int cc = 0; cc < kHd / 32; ++cc) {
          uint32_t acc[32];
          if (ok) {
            tc_ld_32x32(t_o + cc * 32, acc);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) acc[c] = 0u;
          }
          if (row_ok) {
#pragma unroll
            for (int u4 = 0; u4 < 4; ++u4) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(acc[8 * u4]), __uint_as_float(acc[8 * u4 + 1]));
              o.y = pack_bf16x2(__uint_as_float(acc[8 * u4 + 2]), __uint_as_float(acc[8 * u4 + 3]));
              o.z = pack_bf16x2(__uint_as_float(acc[8 * u4 + 4]), __uint_as_float(acc[8 * u4 + 5]));
              o.w = pack_bf16x2(__uint_as_float(acc[8 * u4 + 6]), __uint_as_float(acc[8 * u4 + 7]));
              *reinterpret_cast<uint4*>(orow + cc * 32 + u4 * 8) = o;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(bar_o_empty);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *s_abort && status != nullptr) atomicExch(status, kStatusTimeout);
  if (warp == kSoftWarps + 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512)
                 : "memory");
  }
}

}  // namespace

cudaError_t launch_rope(void* x, const void* pos, int pos64, int64_t rows, int heads, int hd,
                        int dtype, cudaStream_t s) {
  const int64_t total = rows * heads * (hd / 4);
  if (total == 0) return cudaSuccess;
  const unsigned grid = (unsigned)((total + 255) / 256);
  if (dtype)
    rope_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)x, pos, pos64, rows, heads, hd);
  else
    rope_kernel<float><<<grid, 256, 0, s>>>((float*)x, pos, pos64, rows, heads, hd);
  return cudaGetLastError();
}

size_t attention_workspace_bytes(int64_t B, int64_t T) {
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const int64_t Tp = (T + 7) / 8 * 8;
  return 256 + up((size_t)B * T * sizeof(int)) + up((size_t)B * kHd * Tp * 2);
}

bool attention_supported(int dtype, int hd, int64_t B, int64_t T, int N) {
  return dtype == 1 && hd == kHd && B >= 1 && T >= 1 && N >= 1 && T < ((int64_t)1 << 30) &&
         B * N * ((T + kTq - 1) / kTq) < ((int64_t)1 << 31);
}

// q [B,T,N,256] and k [B,T,256] already rotated, v [B,T,256]; out [B,T,N*256].
cudaError_t launch_attention_prefill(const void* q, const void* k, const void* v, const void* pos,
                                     int pos64, int64_t B, int64_t T, int N, int window, void* out,
                                     void* ws, cudaStream_t s) {
  using T_ = __nv_bfloat16;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  const int64_t Tp = (T + 7) / 8 * 8;
  char* base = static_cast<char*>(ws);
  int* status = reinterpret_cast<int*>(base);
  int* lo = reinterpret_cast<int*>(base + 256);
  T_* vt = reinterpret_cast<T_*>(base + 256 + up((size_t)B * T * sizeof(int)));
  attn_bounds_kernel<<<(unsigned)((B + 3) / 4), 128, 0, s>>>(pos, pos64, (int)B, (int)T, window, lo);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  transpose_v_kernel<<<dim3((unsigned)((Tp + 31) / 32), kHd / 32, (unsigned)B), dim3(32, 8), 0, s>>>(
      (const T_*)v, (int)T, (int)Tp, vt);
  if ((err = cudaGetLastError()) != cudaSuccess) return err;
  CUtensorMap map_q, map_k, map_vt;
  if (!tensor_map_bte(&map_q, q, (uint64_t)B, (uint64_t)T, (uint64_t)N * kHd, kTq, kSl, true) ||
      !tensor_map_bte(&map_k, k, (uint64_t)B, (uint64_t)T, kHd, kTk, kSl, true) ||
      !tensor_map_bte(&map_vt, vt, (uint64_t)B, kHd, (uint64_t)Tp, kHd, kSl, true))
    return cudaErrorInvalidValue;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemA);
  }
  const int q_tiles = (int)((T + kTq - 1) / kTq);
  const int n_units = (int)(B * N * q_tiles);
  const int grid = n_units < num_sms ? n_units : num_sms;
  attn_prefill_kernel<<<grid, kThreadsA, kSmemA, s>>>(map_q, map_k, map_vt, lo, (int)B, (int)T, N,
                                                      window, n_units, (T_*)out, status);
  return cudaGetLastError();
}

}  // namespace rgk
