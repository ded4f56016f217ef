// RG-LRU forward in ONE kernel: block-diagonal gate projections on tcgen05, gate arithmetic, and the
// linear recurrence with its cross-tile carry, all in the epilogue, so that the recurrence
// coefficients a and the normalised input never reach HBM (recurrentgemma torch/layers.py:127-137,
// 313-365, 140-191; optional join of torch/modules.py:627-628, 646).  bfloat16, heads of width 256,
// sequence length a multiple of 128.
//
// Units of work: 128 consecutive tokens of one sequence x one half of a head (128 channels, i.e.
// a 256-column accumulator holding the x-gate and the a-gate of those channels).  Units are numbered
// time-major (all sequences and head halves of time tile 0, then of time tile 1, ...) and dealt out
// round-robin to persistent CTAs, one per SM, so that the unit that produces a carry has normally
// finished one round before the unit that consumes it starts.
//
// Per unit: TMA streams the A operand (conv output, 4 K-slices of 128 x 64) and the packed gate
// weights (4 K-slices of 256 x 64) through a 3-stage ring; one thread issues 16 tcgen05.mma into
// one of two TMEM accumulators; 16 epilogue warps (8 per accumulator: 4 row quarters x 2 channel
// halves) drain the other.  An epilogue warp owns 32 tokens x 64 channels and works in chunks of
// 32 channels:
//   row phase    thread = token: tcgen05.ld, gate arithmetic with the reference's bfloat16
//                roundings, (a, x) staged in the warp's 4 KiB of shared memory;
//   column phase lane = channel: the 32 tokens as an affine map (P, H), h -> P h + H; the four row
//                quarters meet at a 128-thread named barrier; the last quarter publishes the
//                tile's map, resolves the incoming state (decoupled look-back over the records of
//                earlier time tiles, normally one already inclusive record) and publishes the
//                inclusive state; second named barrier; every quarter replays its 32 tokens from
//                the staged values with the true incoming state and leaves y in the staging area;
//   row phase    16-byte pieces of y, joined with the other branch, stored 64 contiguous bytes per
//                row and instruction.
// All waits (mbarriers, look-back flags) are bounded; on expiry WsHeader::status is raised, the
// carry of that chunk is taken as zero and the kernel runs to completion.
#include <cuda.h>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tc_common.cuh"

namespace rgk {
namespace {

constexpr int kHW = 256;                 // head width = K
constexpr int kUM = 128;                 // tokens per unit
constexpr int kUN = 256;                 // accumulator columns (128 x-gate + 128 a-gate)
constexpr int kUC = 128;                 // channels per unit
constexpr int kKB = 64;                  // K per ring stage
constexpr int kKBlocks = kHW / kKB;      // 4
constexpr int kRing = 3;
constexpr int kABytesF = kUM * kKB * 2;  // 16 KiB
constexpr int kBBytesF = kUN * kKB * 2;  // 32 KiB
constexpr int kStageF = kABytesF + kBBytesF;
constexpr int kEpiF = 16;
constexpr int kThreadsF = (kEpiF + 2) * 32;
constexpr int kChunk = 32;               // channels per chunk
constexpr int kPlane = 32 * 64;          // one staged tensor of a chunk: 32 rows x 32 bf16
constexpr int kOffRingF = 0;
constexpr int kOffPlanes = kRing * kStageF;                         // 147456: per warp a-plane + x-plane
constexpr int kOffQmap = kOffPlanes + kEpiF * 2 * kPlane;           // float2 [2 acc][2 half][2 chunk][4 q][32]
constexpr int kOffHin = kOffQmap + 2 * 2 * 2 * 4 * 32 * 8;          // float  [2 acc][2 half][2 chunk][32]
constexpr int kOffBarF = kOffHin + 2 * 2 * 2 * 32 * 4;
constexpr int kNumBarF = 2 * kRing + 4;
constexpr int kOffTmemF = kOffBarF + kNumBarF * 8;
constexpr int kOffAbortF = kOffTmemF + 4;
constexpr int kSmemF = kOffAbortF + 4 + 1024;
static_assert(kSmemF <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");
constexpr uint32_t kIdescF = tc_idesc_bf16(kUM, kUN);
constexpr unsigned kLookbackSpins = 1u << 20;

// Look-back record of one (unit, channel half, chunk): 32 channels.
struct ChunkRecord {
  float P[kChunk];
  float H[kChunk];
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ float gelu_fast_f(float z) {
  constexpr float k0 = -1.5957691216057308f * 1.4426950408889634f;
  constexpr float k1 = k0 * 0.044715f;
  const float w = z * fmaf(z * z, k1, k0);
  return z * rcpf(ex2f(w) + 1.0f);
}

// Address of the 16-byte piece `piece` of row r inside a 32 x 64-byte plane (pieces XOR-swizzled by
// row pair: conflict free for row-wise 16-byte and for column-wise 2-byte access).
__device__ __forceinline__ int plane_off(int r, int piece) {
  return r * 64 + ((piece ^ ((r >> 1) & 3)) << 4);
}

template <int kJoin>   // 0: out = y, 1: out = y * gelu_tanh(yb), 2: out = y * yb
__global__ void __launch_bounds__(kThreadsF, 1)
rglru_fused_kernel(const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_w,
                   const __nv_bfloat16* __restrict__ c, const void* __restrict__ pos, int pos64,
                   const __nv_bfloat16* __restrict__ bias_x, const __nv_bfloat16* __restrict__ bias_a,
                   const __nv_bfloat16* __restrict__ m8sp, const float* __restrict__ h0,
                   const __nv_bfloat16* __restrict__ yb, int B, int T_, int E, int groups,
                   int n_units, __nv_bfloat16* __restrict__ out, float* __restrict__ h_last,
                   WsHeader* hdr, unsigned* flags, ChunkRecord* agg, float* incl) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar0 = s_base + kOffBarF;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kRing + s); };
  auto bar_acc_full = [&](int s) { return bar0 + 8u * (2 * kRing + s); };
  auto bar_acc_empty = [&](int s) { return bar0 + 8u * (2 * kRing + 2 + s); };
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + kOffTmemF);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffAbortF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_t = T_ / kUM;
  const int per_tt = B * groups;                         // units per time tile
  const int n_my = (n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int s = 0; s < kRing; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(bar_acc_full(s), 1); mbar_init(bar_acc_empty(s), kEpiF / 2); }
    mbar_fence_init();
  }
  if (warp == kEpiF + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(s_base + kOffTmemF), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == kEpiF) {
    // ------------------------------ TMA producer --------------------------------------------------
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int t = 0; t < n_my && ok; ++t) {
        const int u = blockIdx.x + t * gridDim.x;
        const int tt = u / per_tt, rem = u - tt * per_tt;
        const int b = rem / groups, grp = rem - b * groups;
        const int row0 = b * T_ + tt * kUM;
        for (int kb = 0; kb < kKBlocks; ++kb, ++it) {
          const int s = it % kRing;
          ok = mbar_wait(bar_empty(s), ((it / kRing) & 1) ^ 1, s_abort);
          if (!ok) break;
          mbar_expect_tx(bar_full(s), kStageF);
          tma_load_2d(s_base + kOffRingF + s * kStageF, &map_c, (grp >> 1) * kHW + kb * kKB, row0,
                      bar_full(s));
          tma_load_2d(s_base + kOffRingF + s * kStageF + kABytesF, &map_w, kb * kKB, grp * kUN,
                      bar_full(s));
        }
      }
    }
  } else if (warp == kEpiF + 1) {
    // ------------------------------ MMA issue -----------------------------------------------------
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int t = 0; t < n_my && ok; ++t) {
        const int as = t & 1;
        ok = mbar_wait(bar_acc_empty(as), ((t >> 1) & 1) ^ 1, s_abort);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < kKBlocks; ++kb, ++it) {
          const int s = it % kRing;
          ok = mbar_wait(bar_full(s), (it / kRing) & 1, s_abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a0 = s_base + kOffRingF + s * kStageF, b0 = a0 + kABytesF;
#pragma unroll
          for (int ks = 0; ks < kKB / 16; ++ks)
            tc_mma_bf16(tmem_base + as * kUN, smem_desc_sw128(a0 + ks * 32),
                        smem_desc_sw128(b0 + ks * 32), kIdescF, (kb | ks) != 0 ? 1u : 0u);
          tc_commit(bar_empty(s));
        }
        if (ok) tc_commit(bar_acc_full(as));
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------------------------------
    const int as = warp >> 3;                // accumulator = unit parity
    const int q = warp & 3;                  // row quarter: tokens 32 q .. 32 q + 31, TMEM lanes too
    const int hh = (warp >> 2) & 1;          // channel half of the unit: 64 channels
    const int set_id = 1 + as * 2 + hh;      // named barrier of the four quarters of (as, hh)
    uint8_t* plane_a = smem + kOffPlanes + warp * 2 * kPlane;
    uint8_t* plane_x = plane_a + kPlane;
    bool ok = true;
    for (int t = as; t < n_my; t += 2) {
      const int u = blockIdx.x + t * gridDim.x;
      const int tt = u / per_tt, rem = u - tt * per_tt;
      const int b = rem / groups, grp = rem - b * groups;
      const int64_t row = (int64_t)b * T_ + tt * kUM + q * 32 + lane;   // this thread's token
      const int chan_set = (grp >> 1) * kHW + (grp & 1) * kUC + hh * 64;  // first channel of the set
      const bool is_reset = pos_is_zero(pos, pos64, row);
      if (ok) ok = mbar_wait(bar_acc_full(as), (t >> 1) & 1, s_abort);
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * kUN + hh * 64;

#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int e_chunk = chan_set + cc * kChunk;           // first channel of this chunk
        const int64_t rec = ((int64_t)u * 2 + hh) * 2 + cc;   // record of this (unit, half, chunk)
        float2* s_qmap = reinterpret_cast<float2*>(smem + kOffQmap) + (((as * 2 + hh) * 2 + cc) * 4) * 32;
        float* s_hin = reinterpret_cast<float*>(smem + kOffHin) + ((as * 2 + hh) * 2 + cc) * 32;

        // the last quarter looks at its predecessor's record early: normally it is inclusive already
        float hin_pref = 0.0f;
        bool have_hin = tt == 0;
        if (q == 3) {
          if (tt == 0) {
            hin_pref = h0 != nullptr ? h0[(int64_t)b * E + e_chunk + lane] : 0.0f;
          } else {
            const int64_t rp = rec - (int64_t)per_tt * 4;
            unsigned f = 0;
            if (lane == 0) f = ld_acquire_u32(&flags[rp]);
            f = __shfl_sync(0xffffffffu, f, 0);
            if (f == 2u) {
              __syncwarp();
              hin_pref = ld_cg_f32(incl + rp * kChunk + lane);
              have_hin = true;
            }
          }
        }

        // ---- row phase: gate arithmetic, 16 columns at a time -------------------------------------
        uint4 cv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) cv[j] = *reinterpret_cast<const uint4*>(c + row * E + e_chunk + j * 8);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t zx[16], za[16];
          if (ok) {
            tc_ld_32x16(t_row + cc * kChunk + half * 16, zx);
            tc_ld_32x16(t_row + kUC + cc * kChunk + half * 16, za);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) { zx[i] = 0u; za[i] = 0u; }
          }
#pragma unroll
          for (int j = 0; j < 2; ++j) {                  // 8 channels per 16-byte piece
            const uint4 cw = cv[half * 2 + j];
            const uint32_t cp[4] = {cw.x, cw.y, cw.z, cw.w};
            uint32_t ap[4], xp[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              const int n = j * 8 + p * 2;                // column inside this group of 16
              const int e = e_chunk + half * 16 + n;
              gate_pair(__uint_as_float(zx[n]), __uint_as_float(zx[n + 1]), __uint_as_float(za[n]),
                        __uint_as_float(za[n + 1]), __ldg(reinterpret_cast<const uint32_t*>(bias_x + e)),
                        __ldg(reinterpret_cast<const uint32_t*>(bias_a + e)),
                        __ldg(reinterpret_cast<const uint32_t*>(m8sp + e)), cp[p], is_reset, ap[p],
                        xp[p]);
            }
            const int piece = half * 2 + j;
            *reinterpret_cast<uint4*>(plane_a + plane_off(lane, piece)) = make_uint4(ap[0], ap[1], ap[2], ap[3]);
            *reinterpret_cast<uint4*>(plane_x + plane_off(lane, piece)) = make_uint4(xp[0], xp[1], xp[2], xp[3]);
          }
        }
        if (cc == 1) {
          // both chunks have left TMEM: the accumulator may be overwritten
          tc_fence_before();
          __syncwarp();
          if (lane == 0 && ok) mbar_arrive(bar_acc_empty(as));
        }
        // the join's other factor for the final row phase, in flight during the column phase
        uint4 mv[4];
        if constexpr (kJoin != 0) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int r = (lane >> 2) + 8 * k;
            const int64_t grow = (int64_t)b * T_ + tt * kUM + q * 32 + r;
            mv[k] = ld_stream(yb + grow * E + e_chunk + (lane & 3) * 8);
          }
        }
        __syncwarp();

        // ---- column phase 1: lane = channel, this quarter's 32 tokens as the map (P, H) -----------
        const int col_piece = lane >> 3, col_in = (lane & 7) * 2;
        float P = 1.0f, Hh = 0.0f;
#pragma unroll 8
        for (int r = 0; r < 32; ++r) {
          const int off = plane_off(r, col_piece) + col_in;
          const float av = __uint_as_float((uint32_t)(*reinterpret_cast<const uint16_t*>(plane_a + off)) << 16);
          const float xv = __uint_as_float((uint32_t)(*reinterpret_cast<const uint16_t*>(plane_x + off)) << 16);
          Hh = fmaf(av, Hh, xv);
          P *= av;
        }
        s_qmap[q * 32 + lane] = make_float2(P, Hh);
        named_bar_sync(set_id, 128);

        // ---- the last quarter: publish the tile's map, resolve and publish the incoming state -----
        if (q == 3) {
          float Pt = 1.0f, Ht = 0.0f;
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) {
            const float2 m = s_qmap[qq * 32 + lane];
            Ht = fmaf(m.x, Ht, m.y);
            Pt *= m.x;
          }
          float hin = hin_pref;
          if (tt > 0) {
            agg[rec].P[lane] = Pt;
            agg[rec].H[lane] = Ht;
            __syncwarp();
            if (lane == 0) st_release_u32(&flags[rec], 1u);
            if (!have_hin && ok) {
              // decoupled look-back: lane l polls the flag of the l-th earlier time tile
              float Pc = 1.0f, Hc = 0.0f;
              int base = tt - 1;
              bool done = false, timed_out = false;
              while (!done) {
                const int pred = base - lane;
                const int64_t rp = rec - (int64_t)(tt - pred) * per_tt * 4;
                unsigned f = 2u;
                int L = 32;
                unsigned spins = 0;
                while (true) {
                  if (pred >= 0) f = ld_acquire_u32(&flags[rp]);
                  const unsigned im = __ballot_sync(0xffffffffu, f == 2u);
                  L = im ? (__ffs(im) - 1) : 32;
                  const unsigned need = (L >= 31) ? 0xffffffffu : ((2u << L) - 1u);
                  if ((__ballot_sync(0xffffffffu, f == 0u) & need) == 0u) break;
                  if (++spins > kLookbackSpins) { timed_out = true; break; }
                  __nanosleep(32);
                }
                if (timed_out) break;
                __syncwarp();
                const int n_agg = L < 32 ? L : 32;
                // records are fetched eight at a time, all loads before the first use: the walk
                // costs about one L2 round trip per eight predecessors instead of one each
                for (int j0 = 0; j0 < n_agg; j0 += 8) {
                  float pj[8], hj[8];
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const int j = min(j0 + i, n_agg - 1);
                    const int64_t r2 = rec - (int64_t)(tt - (base - j)) * per_tt * 4;
                    pj[i] = ld_cg_f32(agg[r2].P + lane);
                    hj[i] = ld_cg_f32(agg[r2].H + lane);
                  }
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    if (j0 + i < n_agg) {
                      Hc = fmaf(Pc, hj[i], Hc);
                      Pc *= pj[i];
                    }
                  }
                }
                if (L < 32) {
                  const int64_t r2 = rec - (int64_t)(tt - (base - L)) * per_tt * 4;
                  hin = fmaf(Pc, ld_cg_f32(incl + r2 * kChunk + lane), Hc);
                  done = true;
                } else {
                  base -= 32;
                }
              }
              if (timed_out) {
                if (lane == 0) atomicExch(&hdr->status, kStatusTimeout);
                hin = 0.0f;
              }
            }
          }
          s_hin[lane] = hin;
          const float h_end = fmaf(Pt, hin, Ht);
          incl[rec * kChunk + lane] = h_end;
          if (h_last != nullptr && tt == tiles_t - 1) h_last[(int64_t)b * E + e_chunk + lane] = h_end;
          __syncwarp();
          if (lane == 0) st_release_u32(&flags[rec], 2u);
        }
        named_bar_sync(set_id, 128);

        // ---- column phase 2: replay with the true incoming state; y replaces x in the plane ---------
        {
          float h = s_hin[lane];
          for (int qq = 0; qq < q; ++qq) {
            const float2 m = s_qmap[qq * 32 + lane];
            h = fmaf(m.x, h, m.y);
          }
#pragma unroll 8
          for (int r = 0; r < 32; ++r) {
            const int off = plane_off(r, col_piece) + col_in;
            const float av = __uint_as_float((uint32_t)(*reinterpret_cast<const uint16_t*>(plane_a + off)) << 16);
            const float xv = __uint_as_float((uint32_t)(*reinterpret_cast<const uint16_t*>(plane_x + off)) << 16);
            h = fmaf(av, h, xv);
            *reinterpret_cast<__nv_bfloat16*>(plane_x + off) = __float2bfloat16_rn(h);
          }
        }
        __syncwarp();

        // ---- row phase: join and store, 8 rows x 64 contiguous bytes per instruction ---------------
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int r = (lane >> 2) + 8 * k, piece = lane & 3;
          uint4 yv = *reinterpret_cast<const uint4*>(plane_x + plane_off(r, piece));
          if constexpr (kJoin == 1) {
            const uint32_t mw[4] = {mv[k].x, mv[k].y, mv[k].z, mv[k].w};
            uint32_t yw[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
            for (int p = 0; p < 4; ++p)
              yw[p] = bmul2(yw[p], pack_bf16x2(gelu_fast_f(bf16_lo(mw[p])), gelu_fast_f(bf16_hi(mw[p]))));
            yv = make_uint4(yw[0], yw[1], yw[2], yw[3]);
          } else if constexpr (kJoin == 2) {
            yv = make_uint4(bmul2(yv.x, mv[k].x), bmul2(yv.y, mv[k].y), bmul2(yv.z, mv[k].z),
                            bmul2(yv.w, mv[k].w));
          }
          const int64_t grow = (int64_t)b * T_ + tt * kUM + q * 32 + r;
          *reinterpret_cast<uint4*>(out + grow * E + e_chunk + piece * 8) = yv;
        }
        __syncwarp();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *s_abort) atomicExch(&hdr->status, kStatusTimeout);
  if (warp == kEpiF + 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512)
                 : "memory");
  }
}

// -8 softplus(a_param), rounded as the reference rounds its factors, one value per channel.
__global__ void m8sp_kernel(const __nv_bfloat16* __restrict__ a_param, int E,
                            __nv_bfloat16* __restrict__ m8sp) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < E) {
    const float s = round_bf16(softplus_(__bfloat162float(a_param[e])));
    m8sp[e] = __float2bfloat16_rn(-8.0f * s);
  }
}

bool make_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {kKB, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct FusedLayout {
  int64_t n_units, n_rec;
  size_t flags_off, m8sp_off, agg_off, incl_off, total;
};

FusedLayout fused_layout(int64_t B, int64_t T, int64_t E) {
  FusedLayout L;
  const int64_t groups = E / kUC;
  L.n_units = (T / kUM) * B * groups;
  L.n_rec = L.n_units * 4;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  L.flags_off = sizeof(WsHeader);
  L.m8sp_off = up(L.flags_off + (size_t)L.n_rec * sizeof(unsigned));
  L.agg_off = up(L.m8sp_off + (size_t)E * 2);
  L.incl_off = up(L.agg_off + (size_t)L.n_rec * sizeof(ChunkRecord));
  L.total = up(L.incl_off + (size_t)L.n_rec * kChunk * sizeof(float));
  return L;
}

}  // namespace

bool rglru_fused_supported(int dtype, int bw, int64_t B, int64_t T) {
  return dtype == 1 && bw == kHW && B >= 1 && T >= kUM && T % kUM == 0 &&
         B * T < ((int64_t)1 << 31);
}

size_t rglru_fused_workspace_bytes(int64_t B, int64_t T, int64_t E) {
  if (T < kUM || T % kUM != 0) return 0;
  return fused_layout(B, T, E).total;
}

cudaError_t launch_rglru_fused(const void* c, const void* pos, int pos64, const void* a_param,
                               const void* bx, const void* ba, const void* packed_w,
                               const float* h0, const void* yb, int y_activated, int64_t B,
                               int64_t T, int H, void* out, float* h_last, void* ws,
                               cudaStream_t s) {
  using T_ = __nv_bfloat16;
  const int E = H * kHW;
  const FusedLayout L = fused_layout(B, T, E);
  char* base = static_cast<char*>(ws);
  // flags start at zero (the status word before them belongs to the caller)
  cudaError_t err = cudaMemsetAsync(base + sizeof(int), 0, L.m8sp_off - sizeof(int), s);
  if (err != cudaSuccess) return err;
  T_* m8sp = reinterpret_cast<T_*>(base + L.m8sp_off);
  m8sp_kernel<<<(E + 255) / 256, 256, 0, s>>>((const T_*)a_param, E, m8sp);
  if ((err = cudaGetLastError()) != cudaSuccess) return err;

  CUtensorMap map_c, map_w;
  if (!make_map_2d(&map_c, c, (uint64_t)(B * T), (uint64_t)E, kUM) ||
      !make_map_2d(&map_w, packed_w, (uint64_t)H * 2 * kUN, kHW, kUN))
    return cudaErrorInvalidValue;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(rglru_fused_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemF);
    cudaFuncSetAttribute(rglru_fused_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemF);
    cudaFuncSetAttribute(rglru_fused_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemF);
  }
  const int groups = 2 * H;
  const int n_units = (int)L.n_units;
  const int grid = n_units < num_sms ? n_units : num_sms;   // all CTAs resident: look-back may spin
#define RGK_FUSED(J)                                                                             \
  rglru_fused_kernel<J><<<grid, kThreadsF, kSmemF, s>>>(                                         \
      map_c, map_w, (const T_*)c, pos, pos64, (const T_*)bx, (const T_*)ba, m8sp, h0,            \
      (const T_*)yb, (int)B, (int)T, E, groups, n_units, (T_*)out, h_last,                       \
      reinterpret_cast<WsHeader*>(base), reinterpret_cast<unsigned*>(base + L.flags_off),        \
      reinterpret_cast<ChunkRecord*>(base + L.agg_off), reinterpret_cast<float*>(base + L.incl_off))
  const int join = yb == nullptr ? 0 : (y_activated ? 2 : 1);
  if (join == 0) RGK_FUSED(0); else if (join == 1) RGK_FUSED(1); else RGK_FUSED(2);
#undef RGK_FUSED
  return cudaGetLastError();
}

}  // namespace rgk
