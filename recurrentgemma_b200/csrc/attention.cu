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
// persistent CTAs.  Roles in a CTA (18 warps):
//   warps 0-15 softmax: group g = (warp / 4) % 2 takes the key tiles of parity g (its own S
//              accumulator); a thread owns a query row (TMEM lane quarter warp % 4) and the 64 keys
//              of column half warp / 8 of every tile of its group.  In pass 2 it writes the rounded
//              probabilities back into tensor memory over the logits it has just read (two
//              bfloat16 per 32-bit column, the layout of an operand A held in tensor memory);
//   warp 16    TMA producer: the query tile once per unit (four slices of 64 of the head dimension,
//              resident for both passes) and the key tiles as slices of 64 into a 5-slot ring;
//   warp 19    TMA producer of the transposed values (two 64-key slices per key tile of pass 2);
//   warp 17    TMEM allocation and issue of S = Q K^T (M 128, N 128, 16 K-steps) into S[parity];
//   warp 18    issue of O += P V (M 128, N 256, 8 K-steps, A = P from tensor memory) once the
//              group has written P.  Two issuing warps, so that a P V never queues behind the
//              sixteen instructions of the next Q K^T; the Q K^T warp waits for the P V that read
//              P from S[parity] before it overwrites S[parity].
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
constexpr int kSlice = kTq * kSl * 2;                // a [128 x 64] bfloat16 slice: 16 KiB
constexpr int kRingK = 5;                            // key slices in flight
constexpr int kVStage = kHd * kSl * 2;               // a 64-key slice of V^T: 32 KiB
constexpr int kOffQ = 0;                             // the query tile, four slices
constexpr int kOffK = (kHd / kSl) * kSlice;          //  65536
constexpr int kOffV = kOffK + kRingK * kSlice;       // 147456
// The partial (max, sum) of a row, float2 [2 groups x 2 column halves][128 rows], exchanged between
// the passes.
constexpr int kOffMl = kOffV + 2 * kVStage;          // 212992
constexpr int kOffBarA = kOffMl + 4 * kTq * 8;       // 217088
constexpr int kNumBarA = 2 + 2 * kRingK + 4 + 8 + 2; // q, key ring, v, s_full/s_empty/p_full/pv_done [2], o
constexpr int kOffTmemA = kOffBarA + kNumBarA * 8;
constexpr int kOffAbortA = kOffTmemA + 4;
constexpr int kSmemA = kOffAbortA + 4 + 1024;
static_assert(kSmemA <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");
constexpr int kSoftWarps = 16;
constexpr int kThreadsA = (kSoftWarps + 4) * 32;
constexpr uint32_t kIdescS = tc_idesc_bf16(kTq, kTk);
constexpr uint32_t kIdescO = tc_idesc_bf16(kTq, kHd);
constexpr float kNegBig = -3.0e38f;

// Two floats rounded to bfloat16 and widened again, through the packed conversion (the scalar one
// occupies the special-function pipe that the exponentials need).
__device__ __forceinline__ void round2_bf16(float a, float b, float& ra, float& rb) {
  const uint32_t pk = pack_bf16x2(a, b);
  ra = __uint_as_float(pk << 16);
  rb = __uint_as_float(pk & 0xffff0000u);
}

__global__ void __launch_bounds__(kThreadsA, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_vt, const int* __restrict__ lo_all, int B,
                    int T_, int N, int window, int n_units, __nv_bfloat16* __restrict__ out,
                    int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar0 = s_base + kOffBarA;
  const uint32_t bar_q_full = bar0, bar_q_empty = bar0 + 8u;
  auto bar_full = [&](int s) { return bar0 + 8u * (2 + s); };
  auto bar_empty = [&](int s) { return bar0 + 8u * (2 + kRingK + s); };
  auto bar_v_full = [&](int s) { return bar0 + 8u * (2 + 2 * kRingK + s); };
  auto bar_v_empty = [&](int s) { return bar0 + 8u * (2 + 2 * kRingK + 2 + s); };
  auto bar_s_full = [&](int g) { return bar0 + 8u * (2 + 2 * kRingK + 4 + g); };
  auto bar_s_empty = [&](int g) { return bar0 + 8u * (2 + 2 * kRingK + 6 + g); };
  auto bar_p_full = [&](int g) { return bar0 + 8u * (2 + 2 * kRingK + 8 + g); };
  auto bar_pv_done = [&](int g) { return bar0 + 8u * (2 + 2 * kRingK + 10 + g); };
  const uint32_t bar_o_full = bar0 + 8u * (2 + 2 * kRingK + 12);
  const uint32_t bar_o_empty = bar0 + 8u * (2 + 2 * kRingK + 13);
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + kOffTmemA);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffAbortA);
  float2* s_ml = reinterpret_cast<float2*>(smem + kOffMl);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (T_ + kTq - 1) / kTq;
  const int n_my = (n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (threadIdx.x == 0) {
    *s_abort = 0;
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_empty, 1);
    for (int s = 0; s < kRingK; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_v_full(s), 1); mbar_init(bar_v_empty(s), 1);
      mbar_init(bar_s_full(s), 1); mbar_init(bar_s_empty(s), 8);
      mbar_init(bar_p_full(s), 8);
      mbar_init(bar_pv_done(s), 1);
    }
    mbar_init(bar_o_full, 1);
    mbar_init(bar_o_empty, 8);
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
    // The whole warp runs the loop and waits; one elected lane issues.
    {
      int slot = 0;
      unsigned slot_phase = 1;
      bool ok = true;
      for (int i = 0; i < n_my && ok; ++i) {
        int b, n, t0, j_lo, j_hi;
        unit_of(i, b, n, t0, j_lo, j_hi);
        // the query tile, once the previous unit's last Q K^T has read the old one
        ok = mbar_wait(bar_q_empty, (i & 1) ^ 1, s_abort);
        if (!ok) break;
        if (elect_one()) {
          mbar_expect_tx(bar_q_full, (kHd / kSl) * kSlice);
#pragma unroll
          for (int ks = 0; ks < kHd / kSl; ++ks)
            tma_load_3d(s_base + kOffQ + ks * kSlice, &map_q, n * kHd + ks * kSl, t0, b, bar_q_full);
        }
        __syncwarp();
        for (int pass = 0; pass < 2 && ok; ++pass) {
          for (int j = j_lo; j <= j_hi && ok; ++j) {
#pragma unroll
            for (int ks = 0; ks < kHd / kSl; ++ks) {
              if (ok) ok = mbar_wait(bar_empty(slot), slot_phase, s_abort);
              if (!ok) break;
              if (elect_one()) {
                mbar_expect_tx(bar_full(slot), kSlice);
                tma_load_3d(s_base + kOffK + slot * kSlice, &map_k, ks * kSl, j * kTk, b,
                            bar_full(slot));
              }
              __syncwarp();
              if (++slot == kRingK) { slot = 0; slot_phase ^= 1; }
            }
          }
        }
      }
    }
  } else if (warp == kSoftWarps + 3) {
    // ------------------------------ TMA producer of V^T -------------------------------------------
    {
      unsigned iv = 0;
      bool ok = true;
      for (int i = 0; i < n_my && ok; ++i) {
        int b, n, t0, j_lo, j_hi;
        unit_of(i, b, n, t0, j_lo, j_hi);
        for (int j = j_lo; j <= j_hi && ok; ++j) {
#pragma unroll
          for (int c = 0; c < kTk / kSl; ++c, ++iv) {
            const int s = iv & 1;
            if (ok) ok = mbar_wait(bar_v_empty(s), ((iv >> 1) & 1) ^ 1, s_abort);
            if (!ok) break;
            if (elect_one()) {
              mbar_expect_tx(bar_v_full(s), kVStage);
              tma_load_3d(s_base + kOffV + s * kVStage, &map_vt, j * kTk + c * kSl, 0, b,
                          bar_v_full(s));
            }
            __syncwarp();
          }
        }
      }
    }
  } else if (warp == kSoftWarps + 1) {
    // ------------------------------ Q K^T issue ---------------------------------------------------
    // The whole warp runs the loop and waits; one elected lane issues.
    {
      int slot = 0;
      unsigned slot_phase = 0;
      unsigned s_use[2] = {0, 0};
      unsigned pv_issued[2] = {0, 0}, pv_seen[2] = {0, 0};   // P V on S[g]: scheduled / waited for
      bool ok = true;
      bool k_ready = false;      // the next key slice was already there when last asked
      auto issue_qk = [&](int g) {
        // S[g] = Q K^T for the next key tile in the ring, once the softmax warps have read the old
        // logits and every P V that takes its probabilities from S[g] has completed
        if (ok) ok = mbar_wait(bar_s_empty(g), (s_use[g] & 1) ^ 1, s_abort);
        ++s_use[g];
        while (ok && pv_seen[g] != pv_issued[g]) {
          ok = mbar_wait(bar_pv_done(g), pv_seen[g] & 1, s_abort);
          ++pv_seen[g];
        }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kHd / kSl; ++ks) {
          // (every lane sees the same barrier state and abort flag, so `ok` stays warp-uniform)
          if (ok && !k_ready) ok = mbar_wait(bar_full(slot), slot_phase, s_abort);
          if (!ok) break;
          tc_fence_after();
          // a K step of 16 bfloat16 is 32 bytes = 2 units of the descriptor's start address
          const uint64_t dq = smem_desc_sw128(s_base + kOffQ + ks * kSlice);
          const uint64_t dk = smem_desc_sw128(s_base + kOffK + slot * kSlice);
          // ask about the slice after this one now; the answer is looked at after the issue
          const int slot_n = slot + 1 == kRingK ? 0 : slot + 1;
          k_ready = mbar_test(bar_full(slot_n), slot_n == 0 ? slot_phase ^ 1 : slot_phase);
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < kSl / 16; ++kk)
              tc_mma_bf16(tmem_base + g * kTk, dq + 2 * kk, dk + 2 * kk, kIdescS,
                          (ks | kk) != 0 ? 1u : 0u);
            tc_commit(bar_empty(slot));
          }
          __syncwarp();
          if (++slot == kRingK) { slot = 0; slot_phase ^= 1; }
        }
        if (ok && elect_one()) tc_commit(bar_s_full(g));
        __syncwarp();
      };
      for (int i = 0; i < n_my; ++i) {
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        int b, n, t0, j_lo, j_hi;
        unit_of(i, b, n, t0, j_lo, j_hi);
        const int nt = j_hi - j_lo + 1;
        ok = mbar_wait(bar_q_full, i & 1, s_abort);
        // pass 1: logits only
        for (int j = 0; j < nt && ok; ++j) issue_qk(j & 1);
        // pass 2: the logits again; the other warp issues P V for tile j once its P is written
        for (int j = 0; j < nt && ok; ++j) {
          issue_qk(j & 1);
          ++pv_issued[j & 1];
        }
        if (ok && elect_one()) tc_commit(bar_q_empty);       // the unit's last Q K^T is in the pipe
        __syncwarp();
      }
    }
  } else if (warp == kSoftWarps + 2) {
    // ------------------------------ P V issue -----------------------------------------------------
    {
      unsigned iv = 0;
      unsigned p_use[2] = {0, 0};
      bool ok = true;
      for (int i = 0; i < n_my; ++i) {
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        int b, n, t0, j_lo, j_hi;
        unit_of(i, b, n, t0, j_lo, j_hi);
        const int nt = j_hi - j_lo + 1;
        // the epilogue has read the previous unit's accumulator
        ok = mbar_wait(bar_o_empty, (i & 1) ^ 1, s_abort);
        tc_fence_after();
        for (int j = 0; j < nt && ok; ++j) {
          // O += P V for the key tile whose probabilities group g has just written over S[g]: the
          // keys of half c are the 32 columns from S[g] + 64 c, 8 columns per K step of 16
          const int g = j & 1;
          ok = mbar_wait(bar_p_full(g), p_use[g] & 1, s_abort);
          ++p_use[g];
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < kTk / kSl; ++c, ++iv) {
            const int s = iv & 1;
            if (ok) ok = mbar_wait(bar_v_full(s), (iv >> 1) & 1, s_abort);
            if (!ok) break;
            tc_fence_after();
            const uint32_t p0 = tmem_base + g * kTk + c * 64;
            const uint64_t dv = smem_desc_sw128(s_base + kOffV + s * kVStage);
            if (elect_one()) {
#pragma unroll
              for (int kk = 0; kk < kSl / 16; ++kk)
                tc_mma_bf16_ts(tmem_base + 2 * kTk, p0 + kk * 8, dv + 2 * kk, kIdescO,
                               (j == 0 && c == 0 && kk == 0) ? 0u : 1u);
              tc_commit(bar_v_empty(s));
            }
            __syncwarp();
          }
          if (ok && elect_one()) tc_commit(bar_pv_done(g));
          __syncwarp();
        }
        if (ok && elect_one()) tc_commit(bar_o_full);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------ softmax and epilogue ------------------------------------------
    const int g = (warp >> 2) & 1, quarter = warp & 3, chalf = warp >> 3;
    const int row = quarter * 32 + lane;                     // query row inside the tile = TMEM lane
    const uint32_t t_s = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + g * kTk + chalf * 64;
    const uint32_t t_o = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + 2 * kTk + chalf * 128;
    constexpr float kScale = 0.0625f * 1.4426950408889634f;  // hd^-1/2 log2(e): exponent per logit unit
    unsigned cs = 0;
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

      // ---- pass 1: row maximum and sum over this thread's keys ------------------------------------
      float m = kNegBig, l = 0.0f;
      for (int j = g; j < nt; j += 2) {
        if (ok) ok = mbar_wait(bar_s_full(g), cs & 1, s_abort);
        ++cs;
        tc_fence_after();
        const int s0 = (j_lo + j) * kTk + chalf * 64;
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
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
          if (sc > hi || sc + 31 < lo) {                    // nothing visible in these 32 keys
#pragma unroll
            for (int c = 0; c < 32; ++c) v[c] = kNegBig;
          } else if (sc >= lo && sc + 31 <= hi) {           // all visible: the common case
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              round2_bf16(__uint_as_float(acc[c]), __uint_as_float(acc[c + 1]), v[c], v[c + 1]);
              cm = fmaxf(cm, fmaxf(v[c], v[c + 1]));
            }
          } else {
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              round2_bf16(__uint_as_float(acc[c]), __uint_as_float(acc[c + 1]), v[c], v[c + 1]);
              if (!(sc + c >= lo && sc + c <= hi)) v[c] = kNegBig;
              if (!(sc + c + 1 >= lo && sc + c + 1 <= hi)) v[c + 1] = kNegBig;
              cm = fmaxf(cm, fmaxf(v[c], v[c + 1]));
            }
          }
          if (cm > kNegBig) {
            const float m_new = fmaxf(m, cm);
            const float off = -m_new * kScale;
            float add = 0.0f;
            // a masked key contributes 2^(-huge) = 0
#pragma unroll
            for (int c = 0; c < 32; ++c) add += ex2f(fmaf(v[c], kScale, off));
            l = l * ex2f(fmaxf((m - m_new) * kScale, -200.0f)) + add;
            m = m_new;
          }
          __syncwarp();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(bar_s_empty(g));
      }
      // the four partial (m, l) of a row -> its final ones
      s_ml[(g * 2 + chalf) * kTq + row] = make_float2(m, l);
      named_bar_sync(1, kSoftWarps * 32);
      {
        float m_all = kNegBig;
#pragma unroll
        for (int k = 0; k < 4; ++k) m_all = fmaxf(m_all, s_ml[k * kTq + row].x);
        float l_all = 0.0f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 o = s_ml[k * kTq + row];
          if (o.x > kNegBig) l_all += o.y * ex2f((o.x - m_all) * kScale);
        }
        m = m_all;
        l = l_all;
      }
      named_bar_sync(1, kSoftWarps * 32);      // the exchange area may be rewritten from here on
      // p = 2^(s k - (m k + log2 l)): the normalisation rides in the exponent
      const float off2 = -(m * kScale + log2f(fmaxf(l, 1e-30f)));

      // ---- pass 2: normalised probabilities, rounded, into P[g] -----------------------------------
      for (int j = g; j < nt; j += 2) {
        if (ok) ok = mbar_wait(bar_s_full(g), cs & 1, s_abort);
        ++cs;
        tc_fence_after();
        const int s0 = (j_lo + j) * kTk + chalf * 64;
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
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
          if (sc >= lo && sc + 31 <= hi) {                  // all visible
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              float s0v, s1v;
              round2_bf16(__uint_as_float(acc[c]), __uint_as_float(acc[c + 1]), s0v, s1v);
              pk[c >> 1] = pack_bf16x2(ex2f(fmaf(s0v, kScale, off2)), ex2f(fmaf(s1v, kScale, off2)));
            }
          } else if (sc > hi || sc + 31 < lo) {             // none visible
#pragma unroll
            for (int c = 0; c < 16; ++c) pk[c] = 0u;
          } else {
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              float s0v, s1v;
              round2_bf16(__uint_as_float(acc[c]), __uint_as_float(acc[c + 1]), s0v, s1v);
              const float p0 = (sc + c >= lo && sc + c <= hi) ? ex2f(fmaf(s0v, kScale, off2)) : 0.0f;
              const float p1 =
                  (sc + c + 1 >= lo && sc + c + 1 <= hi) ? ex2f(fmaf(s1v, kScale, off2)) : 0.0f;
              pk[c >> 1] = pack_bf16x2(p0, p1);
            }
          }
          // 32 keys = 16 columns, over logits this thread has already read
          __syncwarp();
          if (ok) tc_st_32x16(t_s + cc * 16, pk);
        }
        tc_wait_st();
        tc_fence_before();
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
        __nv_bfloat16* orow = out + ((int64_t)b * T_ + t) * ((int64_t)N * kHd) + (int64_t)n * kHd +
                              chalf * 128;
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
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
  static PerDeviceOnce once;
  int num_sms = 0;
  cudaError_t e0 = once.run([] {
    return cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemA);
  }, &num_sms);
  if (e0 != cudaSuccess) return e0;
  const int q_tiles = (int)((T + kTq - 1) / kTq);
  const int n_units = (int)(B * N * q_tiles);
  const int grid = n_units < num_sms ? n_units : num_sms;
  attn_prefill_kernel<<<grid, kThreadsA, kSmemA, s>>>(map_q, map_k, map_vt, lo, (int)B, (int)T, N,
                                                      window, n_units, (T_*)out, status);
  return cudaGetLastError();
}

}  // namespace rgk
