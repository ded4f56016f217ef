// The linear recurrence of the RG-LRU, h_t = a_t h_{t-1} + x_t with a float32 state
// (recurrentgemma torch/layers.py:140-191), as a single-pass chunked parallel scan.
//
// Decomposition.  The [B, T, E] problem is cut into tiles of kRows time steps x 64 channels.
// The x and a tiles are brought into shared memory by TMA (two cp.async.bulk.tensor copies per
// tile, asked for by one thread), so a tile in flight costs no registers and four tiles per SM (three
// in float32) are resident.  Inside a tile every thread owns 4 (8) consecutive time steps of one 16-byte pack of
// channels and runs them sequentially: pass 1 reduces its steps to the pair (P, H) of the affine
// map h -> P h + H, the pairs of the tile's sub-chunks are chained through shared memory, and
// pass 2 replays the same steps from shared memory starting from the now known incoming state.
// Tiles of one sequence are linked by a decoupled look-back: each tile publishes its own (P, H)
// as soon as it has it, then walks back over its predecessors' records (a warp reads up to 32
// flags at a time) until it meets one that already holds the inclusive state.  Tile numbers are
// handed out by an atomic ticket in time-major order, so a predecessor has always started before
// its successor and no tile can wait on one that is not running.  All waits are bounded; a wait
// that expires sets WsHeader::status and the tile continues with a zero carry.
//
// Every input element is read from HBM exactly once and every output written once; the
// other branch's tile (needed once) goes straight to registers.  The optional join with the block's other branch (y * gelu_tanh(y_mul), torch/modules.py:627-628,
// 646) is fused into pass 2.
#include <mutex>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tma.cuh"

namespace rgk {
namespace {

constexpr int kThreads = 256;
constexpr int kChan = 64;        // channels per tile
constexpr unsigned kSpinLimit = 1u << 21;

template <typename T> struct ScanCfg {
  static constexpr int kPack = Traits<T>::kPack;
  // rows a thread scans: 4 (bfloat16), 8 (float32) - a tile is 128 time steps either way, so the
  // chain of tiles a carry travels along is no longer for float32 than for bfloat16
  static constexpr int kRowsPerThread = sizeof(T) == 4 ? 8 : 4;
  static constexpr int kLanesPerRow = kChan / kPack;          // 8 (bf16) or 16 (f32)
  static constexpr int kSubs = kThreads / kLanesPerRow;       // 32 or 16 sub-chunks
  static constexpr int kRows = kSubs * kRowsPerThread;        // 128 time steps per tile
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
__device__ __forceinline__ float2 ld_cg_f2(const void* p) {
  float2 v;
  asm volatile("ld.global.cg.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
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

// Shared memory of one tile (dynamic, 128-byte aligned): the x and a tiles as TMA delivers them
// (row-major, kRows x 64 channels), the per-sub-chunk maps, and a few small arrays.
template <typename T> struct ScanSmem {
  static constexpr int kTileBytes = ScanCfg<T>::kRows * kChan * (int)sizeof(T);      // 16 KiB
  static constexpr int kOffX = 0;
  static constexpr int kOffA = kTileBytes;
  static constexpr int kOffSub = 2 * kTileBytes;                                      // float2 [kSubs][64]
  static constexpr int kOffTile = kOffSub + ScanCfg<T>::kSubs * kChan * 8;            // float2 [64]
  static constexpr int kOffHin = kOffTile + kChan * 8;                                // float [64]
  static constexpr int kOffBar = kOffHin + kChan * 4;                                 // mbarrier
  static constexpr int kOffMisc = kOffBar + 8;                                        // ticket, load ok
  static constexpr int kBytes = kOffMisc + 8 + 128;                                   // + alignment slack
};

template <typename T, int kJoin>   // 0: no join, 1: y * gelu_tanh(y_mul), 2: y * y_mul
__global__ void __launch_bounds__(kThreads, sizeof(T) == 4 ? 3 : 4)
scan_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_a,
            const uint8_t* __restrict__ reset, const void* __restrict__ pos, int pos64,
            const float* __restrict__ h0, const T* __restrict__ y_mul, int B, int T_, int E,
            int tiles_t, int groups, T* __restrict__ y, float* __restrict__ h_last, WsHeader* hdr,
            unsigned* flags, float2* agg, float* incl, unsigned ticket_base, unsigned spin_limit) {
  using Cfg = ScanCfg<T>;
  using Sm = ScanSmem<T>;
  constexpr bool kMul = kJoin != 0;
  constexpr int kPack = Cfg::kPack;
  constexpr bool kBf16 = Traits<T>::kBf16;
  constexpr int kSubs = Cfg::kSubs;
  constexpr int kRowBytes = kChan * (int)sizeof(T);

  extern __shared__ uint8_t smem_raw[];
  // aligned by an offset into the shared array, so that the address space stays known to the
  // compiler (shared-memory load/store instructions instead of generic ones)
  uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
  float2 (*s_sub)[kChan] = reinterpret_cast<float2 (*)[kChan]>(smem + Sm::kOffSub);
  float2* s_tile = reinterpret_cast<float2*>(smem + Sm::kOffTile);
  float* s_hin = reinterpret_cast<float*>(smem + Sm::kOffHin);
  volatile unsigned* s_misc = reinterpret_cast<volatile unsigned*>(smem + Sm::kOffMisc);
  const uint32_t bar = smem_u32(smem + Sm::kOffBar);

  const int tid = threadIdx.x;
  if (tid == 0) {
    s_misc[0] = atomicAdd(&hdr->ticket, 1u) + ticket_base;
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  const unsigned tile = s_misc[0];
  const int nseq = B * groups;
  // extents for the range checks of the checks build
  const int64_t n_tiles_all = (int64_t)tiles_t * nseq, n_act = (int64_t)B * T_ * E;
  (void)n_tiles_all; (void)n_act;
  const int tt = tile / nseq;
  const int seq = tile - tt * nseq;
  const int b = seq / groups;
  const int g = seq - b * groups;
  if (tt >= tiles_t) return;  // cannot happen with the launch grid; keeps indices in range

  // ---- the x and a tiles by TMA: one thread asks, the copy engine delivers both tiles ------------
  // Rows past T and channels past E are zero-filled by the hardware and masked out below.
  if (tid == 0) {
    mbar_expect_tx(bar, 2 * Sm::kTileBytes);
    tma_load_3d(smem_u32(smem + Sm::kOffX), &map_x, g * kChan, tt * Cfg::kRows, b, bar);
    tma_load_3d(smem_u32(smem + Sm::kOffA), &map_a, g * kChan, tt * Cfg::kRows, b, bar);
  }

  const int lane_in_row = tid % Cfg::kLanesPerRow;
  const int sub = tid / Cfg::kLanesPerRow;
  const int e0 = g * kChan + lane_in_row * kPack;
  const bool chan_ok = e0 < E;
  const int t0 = tt * Cfg::kRows + sub * Cfg::kRowsPerThread;
  const int64_t row0 = (int64_t)b * T_;
  unsigned valid = 0, rst = 0;
#pragma unroll
  for (int r = 0; r < Cfg::kRowsPerThread; ++r)
    if (chan_ok && t0 + r < T_) valid |= 1u << r;
  if (reset != nullptr || pos != nullptr) {
    bool rs[Cfg::kRowsPerThread];
#pragma unroll
    for (int r = 0; r < Cfg::kRowsPerThread; ++r) {
      const int64_t row = row0 + min(t0 + r, T_ - 1);
      rs[r] = (reset != nullptr) ? (reset[row] != 0) : pos_is_zero(pos, pos64, row);
    }
#pragma unroll
    for (int r = 0; r < Cfg::kRowsPerThread; ++r) rst |= rs[r] ? (1u << r) : 0u;
  }
  // a_t * !reset_t (torch/layers.py:168) and rows past the end (identity map) in one mask.
  const unsigned live = valid & ~rst;

  // Bounded wait for the tiles.
  {
    bool ok = false;
    for (unsigned i = 0; i < kSpinLimit; ++i) {
      if (mbar_try_wait(bar, 0)) { ok = true; break; }
    }
    if (!ok) {
      if (tid == 0) atomicExch(&hdr->status, kStatusTimeout);
      valid = 0;   // compute nothing from a tile that never arrived; the carries still link up
    }
  }
  const uint8_t* sx = smem + Sm::kOffX + (sub * Cfg::kRowsPerThread) * kRowBytes + lane_in_row * 16;
  const uint8_t* sa = smem + Sm::kOffA + (sub * Cfg::kRowsPerThread) * kRowBytes + lane_in_row * 16;

  // ---- pass 1: this thread's steps as an affine map ----------------------------------------------
  {
    float P[kPack], Hh[kPack];
#pragma unroll
    for (int i = 0; i < kPack; ++i) { P[i] = 1.0f; Hh[i] = 0.0f; }
#pragma unroll
    for (int r = 0; r < Cfg::kRowsPerThread; ++r) {
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
#pragma unroll
    for (int i = 0; i < kPack; ++i) s_sub[sub][lane_in_row * kPack + i] = make_float2(P[i], Hh[i]);
  }
  // The other branch's tile is needed once, in pass 2: it goes straight to registers, and its
  // latency hides behind the carry resolution below.
  uint4 mraw[Cfg::kRowsPerThread];
  if constexpr (kMul) {
    const int e_ld = chan_ok ? e0 : 0;
#pragma unroll
    for (int r = 0; r < Cfg::kRowsPerThread; ++r)
      mraw[r] = ld_stream(y_mul + (row0 + min(t0 + r, T_ - 1)) * E + e_ld);
  }
  __syncthreads();

  // ---- tile aggregate, published before anything is waited for -----------------------------------
  const int64_t rec = (int64_t)tile;  // record index = ticket = tt * nseq + seq
  if (tid < kChan) {
    float P = 1.0f, Hh = 0.0f;
#pragma unroll
    for (int s = 0; s < kSubs; ++s) {
      const float2 ph = s_sub[s][tid];
      Hh = fmaf(ph.x, Hh, ph.y);
      P *= ph.x;
    }
    s_tile[tid] = make_float2(P, Hh);
    if (tt == 0) {
      const int e = g * kChan + tid;
      const float hin = (h0 != nullptr && e < E) ? h0[(int64_t)b * E + e] : 0.0f;
      s_hin[tid] = hin;
      if (RGK_IN_RANGE(rec, n_tiles_all, &hdr->status)) incl[rec * kChan + tid] = fmaf(P, hin, Hh);
    } else {
      if (RGK_IN_RANGE(rec, n_tiles_all, &hdr->status)) agg[rec * kChan + tid] = make_float2(P, Hh);
    }
  }
  // The barrier orders the 64 record stores before thread 0's release store, and a release is
  // cumulative over that order: a tile that acquires the flag sees the whole record.
  __syncthreads();
  if (tid == 0) st_release(&flags[rec], tt == 0 ? 2u : 1u);

  // ---- decoupled look-back by warp 0 (lane owns channels 2*lane, 2*lane+1) -----------------------
  if (tt > 0 && tid < 32) {
    const int lane = tid;
    float Pc0 = 1.0f, Hc0 = 0.0f, Pc1 = 1.0f, Hc1 = 0.0f;
    float hin0 = 0.0f, hin1 = 0.0f;
    int base = tt - 1;
    bool done = false, timed_out = false;
    while (!done) {
      const int pred = base - lane;
      unsigned f = 2u;
      int L = 32;
      unsigned spins = 0;
      while (true) {
        if (pred >= 0 && RGK_IN_RANGE((int64_t)pred * nseq + seq, n_tiles_all, &hdr->status))
          f = ld_acquire(&flags[(int64_t)pred * nseq + seq]);
        const unsigned incl_mask = __ballot_sync(0xffffffffu, f == 2u);
        L = incl_mask ? (__ffs(incl_mask) - 1) : 32;
        const unsigned need = (L >= 31) ? 0xffffffffu : ((2u << L) - 1u);
        const unsigned zero = __ballot_sync(0xffffffffu, f == 0u) & need;
        if (zero == 0u) break;
        if (++spins > spin_limit) { timed_out = true; break; }
        __nanosleep(32);
      }
      if (timed_out) break;
      const int n_agg = L < 32 ? L : 32;  // lanes 0 .. n_agg-1 hold plain aggregates
      for (int j = 0; j < n_agg; ++j) {
        const int64_t r2 = (int64_t)(base - j) * nseq + seq;
        const float4 v = ld_cg_f4(reinterpret_cast<const float4*>(agg + r2 * kChan) + lane);
        Hc0 = fmaf(Pc0, v.y, Hc0); Pc0 *= v.x;
        Hc1 = fmaf(Pc1, v.w, Hc1); Pc1 *= v.z;
      }
      if (L < 32) {
        const int64_t r2 = (int64_t)(base - L) * nseq + seq;
        const float2 v = ld_cg_f2(reinterpret_cast<const float2*>(incl + r2 * kChan) + lane);
        hin0 = fmaf(Pc0, v.x, Hc0);
        hin1 = fmaf(Pc1, v.y, Hc1);
        done = true;
      } else {
        base -= 32;
      }
    }
    if (timed_out) {
      if (lane == 0) atomicExch(&hdr->status, kStatusTimeout);
      hin0 = hin1 = 0.0f;
    }
    s_hin[2 * lane] = hin0;
    s_hin[2 * lane + 1] = hin1;
    const float2 t0v = s_tile[2 * lane], t1v = s_tile[2 * lane + 1];
    float2 inc;
    inc.x = fmaf(t0v.x, hin0, t0v.y);
    inc.y = fmaf(t1v.x, hin1, t1v.y);
    *(reinterpret_cast<float2*>(incl + rec * kChan) + lane) = inc;
    __syncwarp();
    if (lane == 0) st_release(&flags[rec], 2u);
  }
  // ---- the join's factor does not depend on the carry: every warp turns its y_mul rows into
  // round(gelu_tanh(.)) now, so the seven warps that would otherwise sit at the barrier below while
  // warp 0 resolves the carry do most of pass 2's arithmetic in that time ---------------------------
  if constexpr (kJoin == 1) {
#pragma unroll
    for (int r = 0; r < Cfg::kRowsPerThread; ++r) {
      float mv[kPack];
      unpack<T>(mraw[r], mv);
      if constexpr (kBf16) {
        mraw[r] = make_uint4(pack_bf16x2(gelu_fast(mv[0]), gelu_fast(mv[1])),
                             pack_bf16x2(gelu_fast(mv[2]), gelu_fast(mv[3])),
                             pack_bf16x2(gelu_fast(mv[4]), gelu_fast(mv[5])),
                             pack_bf16x2(gelu_fast(mv[6]), gelu_fast(mv[7])));
      } else {
#pragma unroll
        for (int i = 0; i < kPack; ++i) mv[i] = gelu_tanh_<false>(mv[i]);
        mraw[r] = pack<T>(mv);
      }
    }
  }
  __syncthreads();

  // ---- state entering each sub-chunk (kept in place of the sub-chunk's H); the last tile of a
  // sequence also writes h_last -------------------------------------------------------------------
  if (tid < kChan) {
    float h = s_hin[tid];
#pragma unroll
    for (int s = 0; s < kSubs; ++s) {
      const float2 ph = s_sub[s][tid];
      s_sub[s][tid].y = h;
      h = fmaf(ph.x, h, ph.y);
    }
    const int e = g * kChan + tid;
    if (h_last != nullptr && tt == tiles_t - 1 && e < E) h_last[(int64_t)b * E + e] = h;
  }
  __syncthreads();

  // ---- pass 2: replay the tile from shared memory with the true incoming state -------------------
  float h[kPack];
#pragma unroll
  for (int i = 0; i < kPack; ++i) h[i] = s_sub[sub][lane_in_row * kPack + i].y;
#pragma unroll
  for (int r = 0; r < Cfg::kRowsPerThread; ++r) {
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
          yp[0] = mul_bf16x2(yp[0], mraw[r].x);
          yp[1] = mul_bf16x2(yp[1], mraw[r].y);
          yp[2] = mul_bf16x2(yp[2], mraw[r].z);
          yp[3] = mul_bf16x2(yp[3], mraw[r].w);
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
          for (int i = 0; i < kPack; ++i) out[i] = out[i] * mv[i];
        }
        o = pack<T>(out);
      }
      if (RGK_IN_RANGE((row0 + t0 + r) * E + e0, n_act, &hdr->status))
        st_stream(y + (row0 + t0 + r) * E + e0, o);
    }
  }
}

template <typename T, int kJoin>
cudaError_t launch_scan_typed(const void* x, const void* a, const uint8_t* reset, const void* pos,
                              int pos64, const float* h0, const void* y_mul, int64_t B, int64_t T_,
                              int64_t E, int tiles_t, int groups, unsigned grid, void* y,
                              float* h_last, WsHeader* hdr, unsigned* flags, float2* agg, float* incl,
                              unsigned ticket_base, unsigned spin_limit, cudaStream_t s) {
  CUtensorMap map_x, map_a;
  if (!tensor_map_bte(&map_x, x, (uint64_t)B, (uint64_t)T_, (uint64_t)E, ScanCfg<T>::kRows, kChan, false,
                      (int)sizeof(T)) ||
      !tensor_map_bte(&map_a, a, (uint64_t)B, (uint64_t)T_, (uint64_t)E, ScanCfg<T>::kRows, kChan, false,
                      (int)sizeof(T)))
    return cudaErrorInvalidValue;
  static PerDeviceOnce once;
  cudaError_t e = once.run([] {
    return cudaFuncSetAttribute(scan_kernel<T, kJoin>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                ScanSmem<T>::kBytes);
  });
  if (e != cudaSuccess) return e;
  scan_kernel<T, kJoin><<<grid, kThreads, ScanSmem<T>::kBytes, s>>>(
      map_x, map_a, reset, pos, pos64, h0, (const T*)y_mul, (int)B, (int)T_, (int)E, tiles_t, groups,
      (T*)y, h_last, hdr, flags, agg, incl, ticket_base, spin_limit);
  return cudaGetLastError();
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
  L.incl_off = up(L.agg_off + (size_t)L.ntiles * kChan * sizeof(float2));
  L.total = up(L.incl_off + (size_t)L.ntiles * kChan * sizeof(float));
  return L;
}

}  // namespace

size_t scan_workspace_bytes(int64_t B, int64_t T, int64_t E, int dtype) {
  return scan_layout(B, T, E, dtype).total;
}

cudaError_t launch_scan(const void* x, const void* a, const uint8_t* reset, const void* pos,
                        int pos64, const float* h0, const void* y_mul, int y_activated, int64_t B,
                        int64_t T, int64_t E, int dtype, void* y, float* h_last, void* ws,
                        cudaStream_t s, int skip_time_tiles, unsigned spin_limit) {
  if (B == 0 || T == 0 || E == 0) return cudaSuccess;
  const ScanLayout L = scan_layout(B, T, E, dtype);
  char* base = static_cast<char*>(ws);
  // Ticket and flags start every launch at zero (the status word before them belongs to the
  // caller).
  cudaError_t err = cudaMemsetAsync(base + sizeof(int), 0, L.agg_off - sizeof(int), s);
  if (err != cudaSuccess) return err;
  WsHeader* hdr = reinterpret_cast<WsHeader*>(base);
  unsigned* flags = reinterpret_cast<unsigned*>(base + L.flags_off);
  float2* agg = reinterpret_cast<float2*>(base + L.agg_off);
  float* incl = reinterpret_cast<float*>(base + L.incl_off);
  // skip_time_tiles > 0 (the wait-expiry self-test only): the first time tiles of every sequence are
  // never launched, so their successors find no published record and their bounded waits run out.
  const int64_t skipped = (int64_t)skip_time_tiles * B * L.groups;
  if (skipped < 0 || skipped >= L.ntiles) return cudaErrorInvalidValue;
  const unsigned grid = (unsigned)(L.ntiles - skipped);
  const unsigned limit = spin_limit != 0 ? spin_limit : kSpinLimit;
#define RGK_SCAN_LAUNCH(TYPE, JOIN)                                                               \
  launch_scan_typed<TYPE, JOIN>(x, a, reset, pos, pos64, h0, y_mul, B, T, E, L.tiles_t, L.groups, \
                                grid, y, h_last, hdr, flags, agg, incl, (unsigned)skipped, limit, s)
  const int join = y_mul == nullptr ? 0 : (y_activated ? 2 : 1);
  if (dtype) {
    if (join == 0) return RGK_SCAN_LAUNCH(__nv_bfloat16, 0);
    if (join == 1) return RGK_SCAN_LAUNCH(__nv_bfloat16, 1);
    return RGK_SCAN_LAUNCH(__nv_bfloat16, 2);
  }
  if (join == 0) return RGK_SCAN_LAUNCH(float, 0);
  if (join == 1) return RGK_SCAN_LAUNCH(float, 1);
  return RGK_SCAN_LAUNCH(float, 2);
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
