// Block-diagonal gate projections of the RG-LRU on the 5th-generation tensor cores, fused with the
// gate arithmetic (recurrentgemma torch/layers.py:127-137, 338-353), for bfloat16 and heads of
// width 256.
//
//   z_x = c_h W_x[h] + b_x[h],  z_a = c_h W_a[h] + b_a[h]          (tcgen05.mma, fp32 in TMEM)
//   a, xn = gate arithmetic(c, z_x, z_a, softplus(a_param), reset)   (epilogue, from TMEM)
//
// Work decomposition.  A "group" is one head and one half of its channels: the 128 x-gate and the
// 128 a-gate output columns of those channels form one N = 256 accumulator, so that an epilogue
// thread finds both gates of a channel in its own TMEM lane.  A persistent CTA serves one group:
// the group's weights, pre-packed K-major as [256 (n), 256 (k)] bfloat16 = 128 KiB, are brought in
// once by TMA and stay in shared memory; the CTA then walks its share of the 128-token tiles.
// Per tile the A operand (128 tokens x the head's 256 channels, 64 KiB) arrives by TMA in four
// K-slices of 64 channels (128-byte swizzle), each slice is consumed by four
// tcgen05.mma.cta_group::1.kind::f16 instructions (M 128, N 256, K 16) and released for the next
// tile's slice by tcgen05.commit.  The accumulator is double buffered in TMEM (2 x 256 columns), so
// the tensor pipe works on tile i+1 while the epilogue warps drain tile i.
//
// Warp roles (576 threads): warps 0-7 / 8-15 epilogue for even / odd tiles (warp w reads TMEM lanes
// 32 (w % 4) .. and the channel half (w / 4) % 2 of the tile), warp 16 TMA producer, warp 17 TMEM
// allocation and MMA issue.
//
// Every mbarrier wait is bounded; when one expires the CTA raises WsHeader::status, all roles leave
// their loops, TMEM is released and the kernel returns.
#include <cuda.h>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tc_common.cuh"

namespace rgk {
namespace {

constexpr int kHeadWidth = 256;       // K of the contraction = channels per head
constexpr int kTileM = 128;           // tokens per tile
constexpr int kTileN = 256;           // accumulator columns: 128 x-gate + 128 a-gate
constexpr int kHalf = 128;            // channels per group
constexpr int kKSlice = 64;           // channels per TMA slice (128 bytes)
constexpr int kNumSlices = kHeadWidth / kKSlice;
constexpr int kASliceBytes = kTileM * kKSlice * 2;   // 16 KiB
constexpr int kBSliceBytes = kTileN * kKSlice * 2;   // 32 KiB
constexpr int kEpiWarps = 16;
constexpr int kThreadsTc = (kEpiWarps + 2) * 32;

// shared memory map (offsets from a 1024-byte aligned base)
constexpr int kOffB = 0;
constexpr int kOffA = kOffB + kNumSlices * kBSliceBytes;            // 131072
constexpr int kOffConst = kOffA + kNumSlices * kASliceBytes;        // 196608
constexpr int kConstBytes = 3 * (kHalf / 2) * 4;                    // bias_x, bias_a, -8 softplus (bf16x2)
constexpr int kOffBar = kOffConst + kConstBytes;                    // 8-byte aligned
constexpr int kNumBars = 3 * kNumSlices + 1 + 4;                    // a_full[2][4] a_empty[4] b_full acc_full[2] acc_empty[2]
constexpr int kOffTmemPtr = kOffBar + kNumBars * 8;
constexpr int kOffAbort = kOffTmemPtr + 4;
constexpr int kOffStage = (kOffAbort + 4 + 15) & ~15;               // per-warp store staging
constexpr int kStageBytes = 32 * 64;                                // 32 rows x 32 channels
constexpr int kSmemBytes = kOffStage + kEpiWarps * kStageBytes + 1024;  // + slack for the alignment
static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");

constexpr uint32_t kIdesc = tc_idesc_bf16(kTileM, kTileN);

__global__ void __launch_bounds__(kThreadsTc, 1)
gates_tc_kernel(const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_w,
                const __nv_bfloat16* __restrict__ c, const void* __restrict__ pos, int pos64,
                const __nv_bfloat16* __restrict__ a_param, const __nv_bfloat16* __restrict__ bias_x,
                const __nv_bfloat16* __restrict__ bias_a, int64_t M, int E, int tiles,
                int ctas_per_group, __nv_bfloat16* __restrict__ a_out,
                __nv_bfloat16* __restrict__ xn_out, WsHeader* hdr) {
  extern __shared__ uint8_t smem_raw[];
  // aligned by an offset into the shared array, so that the address space stays known to the
  // compiler (shared-memory load/store instructions instead of generic ones)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t s_b = s_base + kOffB, s_a = s_base + kOffA;
  uint32_t* s_const = reinterpret_cast<uint32_t*>(smem + kOffConst);   // [3][64] packed pairs
  const uint32_t bar0 = s_base + kOffBar;
  // "slice k is loaded" has one barrier per tile parity: its waiters (the MMA thread and the
  // epilogue warps of that parity) then see every one of its phases, which a waiter that skips
  // every other tile of a single barrier would not.
  auto bar_a_full = [&](int k, int par) { return bar0 + 8u * (par * kNumSlices + k); };
  auto bar_a_empty = [&](int k) { return bar0 + 8u * (2 * kNumSlices + k); };
  const uint32_t bar_b_full = bar0 + 8u * (3 * kNumSlices);
  auto bar_acc_full = [&](int s) { return bar0 + 8u * (3 * kNumSlices + 1 + s); };
  auto bar_acc_empty = [&](int s) { return bar0 + 8u * (3 * kNumSlices + 3 + s); };
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + kOffTmemPtr);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = blockIdx.x / ctas_per_group;          // (head, half)
  const int slot = blockIdx.x % ctas_per_group;
  const int head = group >> 1, half = group & 1;
  const int chan0 = head * kHeadWidth + half * kHalf;     // first channel of the group
  // tiles slot, slot + ctas_per_group, ... of this group
  const int n_my = (tiles - slot + ctas_per_group - 1) / ctas_per_group;

  if (threadIdx.x == 0) {
    *s_abort = 0;
    // A slice is released by the MMA commit and, for the two slices that hold this group's own
    // channels, by the four epilogue warps that copy their conv values out of it.
    for (int k = 0; k < kNumSlices; ++k) {
      mbar_init(bar_a_full(k, 0), 1);
      mbar_init(bar_a_full(k, 1), 1);
      mbar_init(bar_a_empty(k), (k >> 1) == half ? 5 : 1);
    }
    mbar_init(bar_b_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(bar_acc_full(s), 1); mbar_init(bar_acc_empty(s), kEpiWarps / 2); }
    mbar_fence_init();
  }
  if (warp == kEpiWarps + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(s_base + kOffTmemPtr), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x < 3 * (kHalf / 2)) {
    // per-channel constants as packed pairs: bias_x, bias_a, -8 softplus(a_param)
    const int which = threadIdx.x / (kHalf / 2), pair = threadIdx.x % (kHalf / 2);
    const int e = chan0 + 2 * pair;
    uint32_t v;
    if (which == 0) v = *reinterpret_cast<const uint32_t*>(bias_x + e);
    else if (which == 1) v = *reinterpret_cast<const uint32_t*>(bias_a + e);
    else {
      const float s0 = round_bf16(softplus_(__bfloat162float(a_param[e])));
      const float s1 = round_bf16(softplus_(__bfloat162float(a_param[e + 1])));
      v = pack_bf16x2(-8.0f * s0, -8.0f * s1);
    }
    s_const[which * (kHalf / 2) + pair] = v;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == kEpiWarps) {
    // ------------------------------ TMA producer --------------------------------------------------
    if (lane == 0) {
      mbar_expect_tx(bar_b_full, kNumSlices * kBSliceBytes);
      for (int k = 0; k < kNumSlices; ++k)
        tma_load_2d(s_b + k * kBSliceBytes, &map_w, k * kKSlice, group * kTileN, bar_b_full);
      bool ok = true;
      for (int it = 0; it < n_my && ok; ++it) {
        const int tile = slot + it * ctas_per_group;
        for (int k = 0; k < kNumSlices; ++k) {
          ok = mbar_wait(bar_a_empty(k), (it & 1) ^ 1, s_abort);
          if (!ok) break;
          mbar_expect_tx(bar_a_full(k, it & 1), kASliceBytes);
          tma_load_2d(s_a + k * kASliceBytes, &map_c, head * kHeadWidth + k * kKSlice,
                      tile * kTileM, bar_a_full(k, it & 1));
        }
      }
    }
  } else if (warp == kEpiWarps + 1) {
    // ------------------------------ MMA issue -----------------------------------------------------
    if (lane == 0) {
      bool ok = mbar_wait(bar_b_full, 0, s_abort);
      for (int it = 0; it < n_my && ok; ++it) {
        const int s = it & 1;
        ok = mbar_wait(bar_acc_empty(s), ((it >> 1) & 1) ^ 1, s_abort);
        if (!ok) break;
        tc_fence_after();
        for (int k = 0; k < kNumSlices && ok; ++k) {
          ok = mbar_wait(bar_a_full(k, it & 1), (it >> 1) & 1, s_abort);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < kKSlice / 16; ++ks) {
            const uint64_t da = smem_desc_sw128(s_a + k * kASliceBytes + ks * 32);
            const uint64_t db = smem_desc_sw128(s_b + k * kBSliceBytes + ks * 32);
            tc_mma_bf16(tmem_base + s * kTileN, da, db, kIdesc, (k | ks) != 0 ? 1u : 0u);
          }
          tc_commit(bar_a_empty(k));     // slice k may be overwritten once these MMAs are done
        }
        if (ok) tc_commit(bar_acc_full(s));
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------------------------------
    const int s = warp >> 3;                 // accumulator stage = tile parity
    const int lane_base = (warp & 3) * 32;   // TMEM lanes this warp may read
    const int col_half = (warp >> 2) & 1;    // which 64 of the tile's 128 channels
    bool ok = true;
    for (int it = s; it < n_my && ok; it += 2) {
      const int tile = slot + it * ctas_per_group;
      const int64_t row = (int64_t)tile * kTileM + lane_base + lane;
      const bool row_ok = row < M;
      const bool is_reset = row_ok && pos_is_zero(pos, pos64, row);
      // The conv outputs this thread gates are already on chip: the TMA slice half*2 + col_half of
      // the A operand holds this group's 64 channels of every row.  Row r of a slice is 128 bytes
      // at r * 128 with its 16-byte units XOR-ed by r % 8 (the 128-byte swizzle).
      const int my_slice = half * 2 + col_half;
      ok = mbar_wait(bar_a_full(my_slice, s), (it >> 1) & 1, s_abort);
      if (!ok) break;
      uint4 cv[8];
      {
        const int r = lane_base + lane;
        const uint8_t* a_row_smem = smem + kOffA + my_slice * kASliceBytes + r * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          cv[u] = *reinterpret_cast<const uint4*>(a_row_smem + ((u ^ (r & 7)) << 4));
      }
      // The slice is handed back to the copy engine below.  The values above are not used until
      // after the accumulator wait, so nothing else keeps the loads ahead of the release: the fence
      // makes every lane's loads complete before the warp-level barrier that precedes it.
      __threadfence_block();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_a_empty(my_slice));
      ok = mbar_wait(bar_acc_full(s), (it >> 1) & 1, s_abort);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + s * kTileN +
                             col_half * 64;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t zx[32], za[32];
        tc_ld_32x32(t_row + cc * 32, zx);
        tc_ld_32x32(t_row + kHalf + cc * 32, za);
        uint4 cw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) cw[j] = cv[cc * 4 + j];
        tc_wait_ld();
        uint4 av[4], xv[4];                      // 8 channels per 16-byte piece
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t cp[4] = {cw[j].x, cw[j].y, cw[j].z, cw[j].w};
          uint32_t ap[4], xp[4];
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const int n = j * 8 + p * 2;                 // channel inside this 32-column chunk
            const int pair = (col_half * 64 + cc * 32 + n) >> 1;
            gate_pair(__uint_as_float(zx[n]), __uint_as_float(zx[n + 1]), __uint_as_float(za[n]),
                      __uint_as_float(za[n + 1]), s_const[pair], s_const[kHalf / 2 + pair],
                      s_const[kHalf + pair], cp[p], is_reset, ap[p], xp[p]);
          }
          av[j] = make_uint4(ap[0], ap[1], ap[2], ap[3]);
          xv[j] = make_uint4(xp[0], xp[1], xp[2], xp[3]);
        }
        // A thread holds 64 bytes of its own row, so storing from here would touch 32 rows per
        // instruction, half a sector each.  The warp's 32 x 32 block is transposed through a
        // 2 KiB staging buffer (16-byte pieces XOR-swizzled by row pair: conflict free both ways)
        // so that every store instruction writes 8 rows x 64 contiguous bytes.
        uint8_t* stage = smem + kOffStage + warp * kStageBytes;
        const int64_t tile_row0 = (int64_t)tile * kTileM + lane_base;
        const int chan_chunk = chan0 + col_half * 64 + cc * 32;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(stage + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
                which == 0 ? av[j] : xv[j];
          __syncwarp();
          __nv_bfloat16* dst = which == 0 ? a_out : xn_out;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int r = (lane >> 2) + 8 * k, piece = lane & 3;
            const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 64 +
                                                            ((piece ^ ((r >> 1) & 3)) << 4));
            const int64_t grow = tile_row0 + r;
            if (grow < M)
              *reinterpret_cast<uint4*>(dst + grow * E + chan_chunk + piece * 8) = v;
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(s));
    }
  }

  // ------------------------------ teardown --------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *s_abort) atomicExch(&hdr->status, kStatusTimeout);
  if (warp == kEpiWarps + 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512)
                 : "memory");
  }
}

// Packs the two gate weights [H, 256 (k), 256 (n)] into K-major groups [H, 2, 256 (n'), 256 (k)]:
// rows 0-127 of a group are the x-gate columns of its 128 channels, rows 128-255 the a-gate ones.
__global__ void pack_gate_weights_kernel(const __nv_bfloat16* __restrict__ wx,
                                         const __nv_bfloat16* __restrict__ wa, int H,
                                         __nv_bfloat16* __restrict__ packed) {
  __shared__ __nv_bfloat16 tile[32][33];
  // grid: (k tiles = 8, n' tiles = 8, groups = 2H); block 32 x 8
  const int group = blockIdx.z, head = group >> 1, half = group & 1;
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;          // n' in [0, 256)
  const __nv_bfloat16* src = (n0 < kHalf ? wx : wa) + (int64_t)head * kHeadWidth * kHeadWidth;
  const int chan = half * kHalf + (n0 % kHalf);                    // source column of n' = n0
  for (int r = threadIdx.y; r < 32; r += 8)                        // r walks k, x walks n
    tile[r][threadIdx.x] = src[(int64_t)(k0 + r) * kHeadWidth + chan + threadIdx.x];
  __syncthreads();
  __nv_bfloat16* dst = packed + (int64_t)group * kTileN * kHeadWidth;
  for (int r = threadIdx.y; r < 32; r += 8)                        // r walks n', x walks k
    dst[(int64_t)(n0 + r) * kHeadWidth + k0 + threadIdx.x] = tile[threadIdx.x][r];
}



}  // namespace

size_t gates_tc_packed_bytes(int H) { return (size_t)H * 2 * kTileN * kHeadWidth * 2; }

bool gates_tc_supported(int dtype, int bw, int64_t M) {
  return dtype == 1 && bw == kHeadWidth && M >= 1 && M < ((int64_t)1 << 31);
}

cudaError_t launch_pack_gate_weights(const void* wx, const void* wa, int H, void* packed_w,
                                     cudaStream_t s) {
  using T_ = __nv_bfloat16;
  pack_gate_weights_kernel<<<dim3(kHeadWidth / 32, kTileN / 32, 2 * H), dim3(32, 8), 0, s>>>(
      (const T_*)wx, (const T_*)wa, H, (T_*)packed_w);
  return cudaGetLastError();
}

cudaError_t launch_gates_tc(const void* c, const void* pos, int pos64, const void* a_param,
                            const void* wx, const void* bx, const void* wa, const void* ba,
                            int64_t M, int H, void* packed_w, int packed_ready, void* a_out,
                            void* xn_out, void* ws_header, cudaStream_t s) {
  if (M == 0) return cudaSuccess;
  using T_ = __nv_bfloat16;
  const int E = H * kHeadWidth;
  if (!packed_ready) {
    cudaError_t err = launch_pack_gate_weights(wx, wa, H, packed_w, s);
    if (err != cudaSuccess) return err;
  }

  CUtensorMap map_c, map_w;
  if (!tensor_map_2d(&map_c, c, (uint64_t)M, (uint64_t)E, kTileM, kKSlice, true) ||
      !tensor_map_2d(&map_w, packed_w, (uint64_t)H * 2 * kTileN, kHeadWidth, kTileN, kKSlice, true))
    return cudaErrorInvalidValue;

  static PerDeviceOnce once;
  int num_sms = 0;
  cudaError_t e0 = once.run([] {
    return cudaFuncSetAttribute(gates_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  }, &num_sms);
  if (e0 != cudaSuccess) return e0;
  const int groups = 2 * H;
  const int tiles = (int)((M + kTileM - 1) / kTileM);
  int cpg = num_sms / groups;
  if (cpg < 1) cpg = 1;
  if (cpg > tiles) cpg = tiles;
gates_tc_kernel<<<groups * cpg, kThreadsTc, kSmemBytes, s>>>(
      map_c, map_w, (const T_*)c, pos, pos64, (const T_*)a_param, (const T_*)bx, (const T_*)ba, M, E,
      tiles, cpg, (T_*)a_out, (T_*)xn_out, reinterpret_cast<WsHeader*>(ws_header));
  return cudaGetLastError();
}

}  // namespace rgk
