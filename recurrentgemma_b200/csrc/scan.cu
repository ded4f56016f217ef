// The linear recurrence of the RG-LRU, h_t = a_t h_{t-1} + x_t with a float32 state
// (recurrentgemma torch/layers.py:140-191), as a single-pass chunked parallel scan.
//
// Decomposition.  The [B, T, E] problem is cut into tiles of kRows time steps x 64 channels, and a
// tile belongs to ONE WARP: the eight warps of a block work on eight unrelated tiles and never meet
// at a block-wide barrier, so a warp that waits (for its data, for a predecessor) costs nothing but
// its own slot.  Per tile:
//   * lane 0 takes the tile number from an atomic ticket and asks the copy engine for the x and a
//     tiles (two cp.async.bulk.tensor copies into the warp's 8 KiB of shared memory, completion on
//     the warp's mbarrier); the other branch's tile, needed once, goes straight to registers;
//   * every lane owns 8 consecutive time steps of one 16-byte pack of channels.  Pass 1 reduces
//     them to the pair (P, H) of the affine map h -> P h + H; warp shuffles chain the sub-chunks
//     of the tile (lanes 8 or 16 apart), which gives every lane the map of everything before it
//     in the tile, and the last sub-chunk's lanes the map of the whole tile;
//   * the tile publishes that map at once (record, then st.release.gpu flag), and only then looks
//     back: the warp reads up to 32 predecessor flags at a time until it meets one that already
//     holds an inclusive state, combining the plain maps in between (decoupled look-back);
//   * pass 2 replays the steps from shared memory from the now known incoming state, rounds y,
//     applies the optional join y * gelu_tanh(y_mul) (torch/modules.py:627-628, 646) and stores.
// Tickets are handed out in time-major order, so a predecessor has always started before its
// successor and no tile waits on one that is not running.  All waits are bounded; a wait that
// expires sets WsHeader::status and the tile continues with a zero carry.
//
// Every input element is read from HBM exactly once and every output written once.
#include <cstdlib>
#include <mutex>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tma.cuh"

namespace rgk {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;
constexpr int kChan = 64;         // channels per tile
constexpr int kRowsPerLane = 8;   // consecutive time steps a lane runs sequentially
constexpr unsigned kSpinLimit = 1u << 21;

template <typename T> struct ScanCfg {
  static constexpr int kPack = Traits<T>::kPack;
  static constexpr int kLanesPerRow = kChan / kPack;        // 8 (bf16) or 16 (f32)
  static constexpr int kSubs = 32 / kLanesPerRow;           // 4 or 2 sub-chunks per tile
  static constexpr int kRows = kSubs * kRowsPerLane;        // 32 or 16 time steps per tile
  static constexpr int kRowBytes = kChan * (int)sizeof(T);  // 128 or 256
  static constexpr int kTileBytes = kRows * kRowBytes;      // 4 KiB either way
  // per-warp shared memory: x tile, a tile, mbarrier
  static constexpr int kWarpSmem = 2 * kTileBytes + 128;
  static constexpr int kSmemBytes = kWarpsPerBlock * kWarpSmem + 128;
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_cg_f4(const void* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

// gelu_tanh(z) for the bfloat16 path: z * sigmoid(2u) with the constants pre-multiplied by
// -log2(e), so that it costs 5 float operations and 2 SFU operations.
__device__ __forceinline__ float gelu_fast(float z) {
  constexpr float k0 = -1.5957691216057308f * 1.4426950408889634f;
  constexpr float k1 = k0 * 0.044715f;
  const float z2 = z * z;
  const float w = z * fmaf(z2, k1, k0);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(w));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
  return z * r;
}

// Product of two packed bfloat16 pairs, each lane rounded to nearest even: the same value torch
// produces when it multiplies two bfloat16 tensors.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Look-back record of one tile: the plain map (P, H) per channel, laid out so that the lane owning
// channels [kPack l, kPack l + kPack) moves whole 16-byte words.
struct TileRecord {
  float P[kChan];
  float H[kChan];
};

template <typename T, bool kMul>
__global__ void __launch_bounds__(kThreads, 3)
scan_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_a,
            const uint8_t* __restrict__ reset, const void* __restrict__ pos, int pos64,
            const float* __restrict__ h0, const T* __restrict__ y_mul, int B, int T_, int E,
            int tiles_t, int groups, unsigned ntiles, T* __restrict__ y,
            float* __restrict__ h_last, WsHeader* hdr, unsigned* flags, TileRecord* agg,
            float* incl) {
  using Cfg = ScanCfg<T>;
  constexpr int kPack = Cfg::kPack;
  constexpr bool kBf16 = Traits<T>::kBf16;
  constexpr int kLpr = Cfg::kLanesPerRow;
  constexpr int kRowBytes = Cfg::kRowBytes;
  constexpr unsigned kFull = 0xffffffffu;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) &
                                             ~static_cast<uintptr_t>(127));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* wsm = smem + warp * Cfg::kWarpSmem;
  const uint32_t bar = smem_u32(wsm + 2 * Cfg::kTileBytes);

  // ---- ticket and the tile request ---------------------------------------------------------------
  unsigned tile = 0;
  if (lane == 0) {
    tile = atomicAdd(&hdr->ticket, 1u);
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  tile = __shfl_sync(kFull, tile, 0);
  if (tile >= ntiles) return;   // the last block may hold warps without a tile
  const int nseq = B * groups;
  const int tt = tile / nseq;
  const int seq = tile - tt * nseq;
  const int b = seq / groups;
  const int g = seq - b * groups;
  if (lane == 0) {
    // Rows past T and channels past E are zero-filled by the copy engine and masked out below.
    mbar_expect_tx(bar, 2 * Cfg::kTileBytes);
    tma_load_3d(smem_u32(wsm), &map_x, g * kChan, tt * Cfg::kRows, b, bar);
    tma_load_3d(smem_u32(wsm + Cfg::kTileBytes), &map_a, g * kChan, tt * Cfg::kRows, b, bar);
  }

  const int lir = lane % kLpr;          // which 16-byte pack of the row
  const int sub = lane / kLpr;          // which sub-chunk of the tile
  const int e0 = g * kChan + lir * kPack;
  const bool chan_ok = e0 < E;
  const int t0 = tt * Cfg::kRows + sub * kRowsPerLane;
  const int64_t row0 = (int64_t)b * T_;

  unsigned valid = 0, rst = 0;
#pragma unroll
  for (int r = 0; r < kRowsPerLane; ++r)
    if (chan_ok && t0 + r < T_) valid |= 1u << r;
  if (reset != nullptr || pos != nullptr) {
    bool rs[kRowsPerLane];
#pragma unroll
    for (int r = 0; r < kRowsPerLane; ++r) {
      const int64_t row = row0 + min(t0 + r, T_ - 1);
      rs[r] = (reset != nullptr) ? (reset[row] != 0) : pos_is_zero(pos, pos64, row);
    }
#pragma unroll
    for (int r = 0; r < kRowsPerLane; ++r) rst |= rs[r] ? (1u << r) : 0u;
  }
  // a_t * !reset_t (torch/layers.py:168): a reset step is the map h -> x_t.
  const unsigned live = valid & ~rst;

  // ---- bounded wait for the tiles ------------------------------------------------------------------
  {
    bool ok = false;
    for (unsigned i = 0; i < kSpinLimit; ++i) {
      if (mbar_try_wait(bar, 0)) { ok = true; break; }
    }
    if (!__all_sync(kFull, ok)) {
      if (lane == 0) atomicExch(&hdr->status, kStatusTimeout);
      valid = 0;   // compute nothing from a tile that never arrived; the carries still link up
    }
  }
  const uint8_t* sx = wsm + (sub * kRowsPerLane) * kRowBytes + lir * 16;
  const uint8_t* sa = sx + Cfg::kTileBytes;

  // ---- pass 1: this lane's steps as an affine map --------------------------------------------------
  float P[kPack], Hh[kPack];
#pragma unroll
  for (int i = 0; i < kPack; ++i) { P[i] = 1.0f; Hh[i] = 0.0f; }
#pragma unroll
  for (int r = 0; r < kRowsPerLane; ++r) {
    if (valid & (1u << r)) {
      float av[kPack], xv[kPack];
      unpack<T>(*reinterpret_cast<const uint4*>(sx + r * kRowBytes), xv);
      if (live & (1u << r)) {
        unpack<T>(*reinterpret_cast<const uint4*>(sa + r * kRowBytes), av);
#pragma unroll
        for (int i = 0; i < kPack; ++i) {
          Hh[i] = fmaf(av[i], Hh[i], xv[i]);
          P[i] *= av[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < kPack; ++i) { Hh[i] = xv[i]; P[i] = 0.0f; }
      }
    }
  }
  // ---- chain the sub-chunks: inclusive scan of the maps over lanes kLpr apart ---------------------
#pragma unroll
  for (int d = kLpr; d < 32; d <<= 1) {
#pragma unroll
    for (int i = 0; i < kPack; ++i) {
      const float Pp = __shfl_up_sync(kFull, P[i], d);
      const float Hp = __shfl_up_sync(kFull, Hh[i], d);
      if (lane >= d) {
        Hh[i] = fmaf(P[i], Hp, Hh[i]);   // (this) o (earlier): h -> P (Pp h + Hp) + H
        P[i] *= Pp;
      }
    }
  }
  // The other branch's tile is needed once, in pass 2: it goes straight to registers, and its
  // latency hides behind the carry resolution below.
  uint4 mraw[kRowsPerLane];
  if constexpr (kMul) {
    const int e_ld = chan_ok ? e0 : 0;
#pragma unroll
    for (int r = 0; r < kRowsPerLane; ++r)
      mraw[r] = ld_stream(y_mul + (row0 + min(t0 + r, T_ - 1)) * E + e_ld);
  }

  // ---- publish the tile's map (or, for the first tile of a sequence, its inclusive state) ---------
  // The lanes of the last sub-chunk hold the whole tile's map for their kPack channels.
  const bool owner = sub == Cfg::kSubs - 1;
  const int ch0 = lir * kPack;
  float hin[kPack];
#pragma unroll
  for (int i = 0; i < kPack; ++i) hin[i] = 0.0f;
  const int64_t rec = (int64_t)tile;   // record index = ticket = tt * nseq + seq
  if (tt == 0) {
    if (h0 != nullptr && chan_ok) {
#pragma unroll
      for (int i = 0; i < kPack; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(h0 + (int64_t)b * E + e0 + i);
        hin[i] = v.x; hin[i + 1] = v.y; hin[i + 2] = v.z; hin[i + 3] = v.w;
      }
    }
    if (owner) {
#pragma unroll
      for (int i = 0; i < kPack; i += 4)
        *reinterpret_cast<float4*>(incl + rec * kChan + ch0 + i) =
            make_float4(fmaf(P[i], hin[i], Hh[i]), fmaf(P[i + 1], hin[i + 1], Hh[i + 1]),
                        fmaf(P[i + 2], hin[i + 2], Hh[i + 2]), fmaf(P[i + 3], hin[i + 3], Hh[i + 3]));
    }
  } else if (owner) {
#pragma unroll
    for (int i = 0; i < kPack; i += 4) {
      *reinterpret_cast<float4*>(agg[rec].P + ch0 + i) = make_float4(P[i], P[i + 1], P[i + 2], P[i + 3]);
      *reinterpret_cast<float4*>(agg[rec].H + ch0 + i) = make_float4(Hh[i], Hh[i + 1], Hh[i + 2], Hh[i + 3]);
    }
  }
  // __syncwarp orders the record stores of the owner lanes before lane 0's release store, and a
  // release is cumulative over that order: a tile that acquires the flag sees the whole record.
  __syncwarp();
  if (lane == 0) st_release(&flags[rec], tt == 0 ? 2u : 1u);

  // ---- decoupled look-back --------------------------------------------------------------------------
  // Every lane polls one predecessor flag; lanes 0 .. kLpr-1 then gather the records for their kPack
  // channels (the same channels for every sub-chunk), nearest predecessor first:
  //   h_in = Pc * h_end(predecessor) + Hc.
  if (tt > 0) {
    float Pc[kPack], Hc[kPack];
#pragma unroll
    for (int i = 0; i < kPack; ++i) { Pc[i] = 1.0f; Hc[i] = 0.0f; }
    int base = tt - 1;
    bool done = false, timed_out = false;
    while (!done) {
      const int pred = base - lane;
      unsigned f = 2u;
      int L = 32;
      unsigned spins = 0;
      while (true) {
        if (pred >= 0) f = ld_acquire(&flags[(int64_t)pred * nseq + seq]);
        const unsigned incl_mask = __ballot_sync(kFull, f == 2u);
        L = incl_mask ? (__ffs(incl_mask) - 1) : 32;
        const unsigned need = (L >= 31) ? kFull : ((2u << L) - 1u);
        const unsigned zero = __ballot_sync(kFull, f == 0u) & need;
        if (zero == 0u) break;
        if (++spins > kSpinLimit) { timed_out = true; break; }
        __nanosleep(32);
      }
      if (timed_out) break;
      // Each flag was acquired by the lane that polled it; the barrier extends that order to the
      // lanes that read the records.
      __syncwarp();
      const int n_agg = L < 32 ? L : 32;   // predecessors base .. base-n_agg+1 hold plain maps
      if (lane < kLpr) {
        for (int j = 0; j < n_agg; ++j) {
          const TileRecord* r2 = agg + ((int64_t)(base - j) * nseq + seq);
#pragma unroll
          for (int i = 0; i < kPack; i += 4) {
            const float4 p4 = ld_cg_f4(r2->P + ch0 + i);
            const float4 h4 = ld_cg_f4(r2->H + ch0 + i);
            Hc[i] = fmaf(Pc[i], h4.x, Hc[i]); Pc[i] *= p4.x;
            Hc[i + 1] = fmaf(Pc[i + 1], h4.y, Hc[i + 1]); Pc[i + 1] *= p4.y;
            Hc[i + 2] = fmaf(Pc[i + 2], h4.z, Hc[i + 2]); Pc[i + 2] *= p4.z;
            Hc[i + 3] = fmaf(Pc[i + 3], h4.w, Hc[i + 3]); Pc[i + 3] *= p4.w;
          }
        }
        if (L < 32) {
          const float* r2 = incl + ((int64_t)(base - L) * nseq + seq) * kChan + ch0;
#pragma unroll
          for (int i = 0; i < kPack; i += 4) {
            const float4 v = ld_cg_f4(r2 + i);
            hin[i] = fmaf(Pc[i], v.x, Hc[i]);
            hin[i + 1] = fmaf(Pc[i + 1], v.y, Hc[i + 1]);
            hin[i + 2] = fmaf(Pc[i + 2], v.z, Hc[i + 2]);
            hin[i + 3] = fmaf(Pc[i + 3], v.w, Hc[i + 3]);
          }
        }
      }
      if (L < 32) done = true; else base -= 32;
    }
    if (timed_out) {
      if (lane == 0) atomicExch(&hdr->status, kStatusTimeout);
#pragma unroll
      for (int i = 0; i < kPack; ++i) hin[i] = 0.0f;
    }
    // hand the incoming state to every sub-chunk's lanes
#pragma unroll
    for (int i = 0; i < kPack; ++i) hin[i] = __shfl_sync(kFull, hin[i], lir);
  }
  // State at the end of this lane's sub-chunk; for the last sub-chunk that is the tile's inclusive
  // state.  The state entering a sub-chunk is the end state of the one before it.
  float h[kPack];
#pragma unroll
  for (int i = 0; i < kPack; ++i) {
    const float h_end = fmaf(P[i], hin[i], Hh[i]);
    P[i] = h_end;                                   // P is not needed any more: reuse as h_end
    const float prev = __shfl_up_sync(kFull, h_end, kLpr);
    h[i] = sub == 0 ? hin[i] : prev;
  }
  if (owner && tt > 0) {
#pragma unroll
    for (int i = 0; i < kPack; i += 4)
      *reinterpret_cast<float4*>(incl + rec * kChan + ch0 + i) =
          make_float4(P[i], P[i + 1], P[i + 2], P[i + 3]);
  }
  if (tt > 0) {
    __syncwarp();
    if (lane == 0) st_release(&flags[rec], 2u);
  }
  // The last tile of a sequence also holds the final state.
  if (h_last != nullptr && tt == tiles_t - 1 && owner && chan_ok) {
#pragma unroll
    for (int i = 0; i < kPack; i += 4)
      *reinterpret_cast<float4*>(h_last + (int64_t)b * E + e0 + i) =
          make_float4(P[i], P[i + 1], P[i + 2], P[i + 3]);
  }

  // ---- pass 2: replay the lane's steps from shared memory with the true incoming state ------------
#pragma unroll
  for (int r = 0; r < kRowsPerLane; ++r) {
    if (valid & (1u << r)) {
      float av[kPack], xv[kPack];
      unpack<T>(*reinterpret_cast<const uint4*>(sx + r * kRowBytes), xv);
      if (live & (1u << r)) {
        unpack<T>(*reinterpret_cast<const uint4*>(sa + r * kRowBytes), av);
#pragma unroll
        for (int i = 0; i < kPack; ++i) h[i] = fmaf(av[i], h[i], xv[i]);
      } else {
#pragma unroll
        for (int i = 0; i < kPack; ++i) h[i] = xv[i];
      }
      uint4 o;
      if constexpr (kBf16) {
        // y = bf16(h); the join multiplies it by bf16(gelu(y_mul)) and rounds once more.
        uint32_t yp[4] = {pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]),
                          pack_bf16x2(h[4], h[5]), pack_bf16x2(h[6], h[7])};
        if constexpr (kMul) {
          float mv[kPack];
          unpack<T>(mraw[r], mv);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            yp[j] = mul_bf16x2(yp[j], pack_bf16x2(gelu_fast(mv[2 * j]), gelu_fast(mv[2 * j + 1])));
        }
        o = make_uint4(yp[0], yp[1], yp[2], yp[3]);
      } else {
        float out[kPack];
#pragma unroll
        for (int i = 0; i < kPack; ++i) out[i] = h[i];
        if constexpr (kMul) {
          float mv[kPack];
          unpack<T>(mraw[r], mv);
#pragma unroll
          for (int i = 0; i < kPack; ++i) out[i] = out[i] * gelu_tanh_<false>(mv[i]);
        }
        o = pack<T>(out);
      }
      st_stream(y + (row0 + t0 + r) * E + e0, o);
    }
  }
}

struct ScanLayout {
  int tiles_t, groups;
  int64_t ntiles;
  size_t flags_off, agg_off, incl_off, total;
};

ScanLayout scan_layout(int64_t B, int64_t T, int64_t E, int dtype) {
  ScanLayout L;
  const int rows = dtype ? ScanCfg<__nv_bfloat16>::kRows : ScanCfg<float>::kRows;
  L.tiles_t = (int)((T + rows - 1) / rows);
  L.groups = (int)((E + kChan - 1) / kChan);
  L.ntiles = (int64_t)L.tiles_t * B * L.groups;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  L.flags_off = sizeof(WsHeader);
  L.agg_off = up(L.flags_off + (size_t)L.ntiles * sizeof(unsigned));
  L.incl_off = up(L.agg_off + (size_t)L.ntiles * sizeof(TileRecord));
  L.total = up(L.incl_off + (size_t)L.ntiles * kChan * sizeof(float));
  return L;
}

// 3-D tensor map over [B, T, E] with a box of kRows x 64 channels of one batch row.
template <typename T>
bool make_scan_map(CUtensorMap* map, const void* base, int64_t B, int64_t T_, int64_t E) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (fn == nullptr) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)E, (cuuint64_t)T_, (cuuint64_t)B};
  const cuuint64_t strides[2] = {(cuuint64_t)E * sizeof(T), (cuuint64_t)T_ * E * sizeof(T)};
  const cuuint32_t box[3] = {kChan, (cuuint32_t)ScanCfg<T>::kRows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = sizeof(T) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  return fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, bool kMul>
cudaError_t launch_scan_typed(const void* x, const void* a, const uint8_t* reset, const void* pos,
                              int pos64, const float* h0, const void* y_mul, int64_t B, int64_t T_,
                              int64_t E, const ScanLayout& L, void* y, float* h_last, char* base,
                              cudaStream_t s) {
  CUtensorMap map_x, map_a;
  if (!make_scan_map<T>(&map_x, x, B, T_, E) || !make_scan_map<T>(&map_a, a, B, T_, E))
    return cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(scan_kernel<T, kMul>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         ScanCfg<T>::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const unsigned grid = (unsigned)((L.ntiles + kWarpsPerBlock - 1) / kWarpsPerBlock);
  scan_kernel<T, kMul><<<grid, kThreads, ScanCfg<T>::kSmemBytes, s>>>(
      map_x, map_a, reset, pos, pos64, h0, (const T*)y_mul, (int)B, (int)T_, (int)E, L.tiles_t,
      L.groups, (unsigned)L.ntiles, (T*)y, h_last, reinterpret_cast<WsHeader*>(base),
      reinterpret_cast<unsigned*>(base + L.flags_off),
      reinterpret_cast<TileRecord*>(base + L.agg_off), reinterpret_cast<float*>(base + L.incl_off));
  return cudaGetLastError();
}

}  // namespace

size_t scan_workspace_bytes(int64_t B, int64_t T, int64_t E, int dtype) {
  return scan_layout(B, T, E, dtype).total;
}

cudaError_t launch_scan(const void* x, const void* a, const uint8_t* reset, const void* pos,
                        int pos64, const float* h0, const void* y_mul, int64_t B, int64_t T,
                        int64_t E, int dtype, void* y, float* h_last, void* ws, cudaStream_t s) {
  if (B == 0 || T == 0 || E == 0) return cudaSuccess;
  const ScanLayout L = scan_layout(B, T, E, dtype);
  char* base = static_cast<char*>(ws);
  // Ticket and flags start every launch at zero (the status word before them belongs to the
  // caller, which clears it once per API call).
  cudaError_t err = cudaMemsetAsync(base + sizeof(int), 0, L.agg_off - sizeof(int), s);
  if (err != cudaSuccess) return err;
#define RGK_SCAN_LAUNCH(TYPE, MUL) \
  launch_scan_typed<TYPE, MUL>(x, a, reset, pos, pos64, h0, y_mul, B, T, E, L, y, h_last, base, s)
  if (dtype) return y_mul ? RGK_SCAN_LAUNCH(__nv_bfloat16, true) : RGK_SCAN_LAUNCH(__nv_bfloat16, false);
  return y_mul ? RGK_SCAN_LAUNCH(float, true) : RGK_SCAN_LAUNCH(float, false);
#undef RGK_SCAN_LAUNCH
}

// ------------------------------------------------------------------------------------------------
// Built-in scratch for callers that may not allocate.
//
// Some hosts of this library own every byte of device memory themselves: a serving runtime that
// plans its buffers once and forbids allocation on the request path, or a process that has handed
// the whole device to its own arena so that a cudaMalloc from a plug-in would simply fail.  Such a
// caller can still pass inputs and outputs, but it has no workspace to lend.  For it the scan can
// run on this array instead, which lives in the library's device image: every GPU that loads
// librgk.so holds these 8 MiB until the process exits.
//
// In host code `g_static_scratch` is only a handle for the symbol, never a device address; the
// address is looked up with cudaGetSymbolAddress, once per device and with that device current.
// ------------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

size_t scan_static_scratch_bytes() { return kStaticScratchBytes; }

cudaError_t scan_static_scratch(void** ptr_out) {
  static std::mutex mu;
  static void* device_ptr[64];
  static int looked_up[64];
  std::lock_guard<std::mutex> lock(mu);
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!looked_up[dev]) {
    void* p = nullptr;
    err = cudaGetSymbolAddress(&p, g_static_scratch);
    if (err != cudaSuccess) return err;
    device_ptr[dev] = p;
    looked_up[dev] = 1;
  }
  *ptr_out = device_ptr[dev];
  return cudaSuccess;
}

}  // namespace rgk
