// Dense projection out = x W^T + b for FEW rows (M <= 256: the decode step, where M is the batch) on
// the 5th-generation tensor cores: torch.nn.Linear as the blocks use it in a decode step
// (recurrentgemma torch/modules.py:437-452, 531-548, 626-647, 749-752).
//
// With so few rows the contraction is bound by streaming the weights (N x K bfloat16, 13 MB at 2B
// dims) exactly once, and the 128 x 256 output tiles of the prefill GEMM would leave most SMs
// without a tile.  Here the WEIGHTS are the tall operand: a CTA owns 128 output features x a slice
// of K and computes the TRANSPOSED tile  D[feature, row] = W_tile x^T  with tcgen05.mma (M 128 =
// features, N = the rows of x rounded up to 16 or 32, K 16): the rows of x are the narrow operand,
// so a pipeline stage is 16 KiB of weights plus only 128 bytes per row of x, and the ring keeps up
// to ten weight tiles in flight per SM - what it takes to cover HBM latency with one CTA per SM.
//
// The K slices of one feature tile are the CTAs of one thread-block cluster (as many as fit the
// GPU in a single wave, at most 8), and their partial sums meet in distributed shared memory: CTA
// r of the cluster finishes the r-th share of the rows of x, every CTA stores its partial sums for
// those rows straight from tensor memory into CTA r's buffer (a lane is a feature, so a warp
// stores 128 contiguous bytes per row), one cluster barrier, and CTA r adds the slices in rank
// order - a fixed order, so the result is the same bits on every run - applies the bias in float32,
// rounds once, applies gelu / residual / GeGLU with their own roundings, and writes its rows of
// the output.  Nothing goes through global scratch.  With a single K slice the epilogue writes
// the output from tensor memory directly.
//
// The kernel is launched with programmatic stream serialisation: its weight fetches start while
// the kernel before it in the stream drains, everything else waits for that kernel's completion.
// Every mbarrier wait is bounded; on expiry the status word (if given) is raised and the CTA goes
// on to the cluster barriers (so its peers are not left waiting) and leaves.
#include <cuda.h>

#include <mutex>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tc_common.cuh"

namespace rgk {
namespace {

constexpr int SN = 128, SK = 64;                  // features per CTA, K per stage
constexpr int kWTile = SN * SK * 2;               // 16 KiB of weights per stage
constexpr int kDataS = 220 * 1024;                // ring + exchange buffer, one CTA per SM
constexpr int kDataHalfS = 109 * 1024;            // the same when two CTAs are to share an SM
constexpr int kMaxStagesS = 10;
constexpr int kMaxClusterS = 8;
constexpr int kEpiS = 8;                          // 4 TMEM lane quarters x 2 column halves
constexpr int kThreadsS = (kEpiS + 2) * 32;
// behind the data: full[] empty[] acc barriers, the TMEM address, the abort flag; 1 KiB to align
constexpr int kOffTmemS = (2 * kMaxStagesS + 1) * 8;
constexpr int kOffAbortS = kOffTmemS + 4;
constexpr int kTailS = 256 + 1024;
static_assert(kOffAbortS + 4 <= 256, "tail too small");
static_assert(kDataS + kTailS <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");
static_assert(2 * (kDataHalfS + kTailS + 1024) <= 233472, "two CTAs do not fit an SM");

// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may
// start while its predecessor in the stream is still running; everything that depends on the
// predecessor's results (and every global write) comes after grid_dependency_wait(), which returns
// once the predecessor has completed and its writes are visible.  Without the attribute both are
// no-ops.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Cluster barrier halves; every thread of every CTA of the cluster executes each of them, warps
// converged (a cluster of one CTA passes at once).
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t peer_smem(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_peer_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float round_bf16(float v) { return bf16_lo(pack_bf16x2(v, 0.0f)); }
__device__ __forceinline__ __nv_bfloat16 bf16_of_rounded(float v) {
  return __ushort_as_bfloat16(static_cast<unsigned short>(__float_as_uint(v) >> 16));
}
__device__ __forceinline__ float bf16_value(__nv_bfloat16 v) {
  return __uint_as_float(static_cast<uint32_t>(__bfloat16_as_ushort(v)) << 16);
}

// One output value from its float32 sum: + bias, one rounding to bfloat16, then (kAct == 1)
// gelu_tanh and a second rounding, then (has_res) the residual add and its rounding - the tensor
// operations of the reference, in its order.
template <int kAct>
__device__ __forceinline__ __nv_bfloat16 finish1(float sum, float bias, bool has_res, float res) {
  float y = round_bf16(sum + bias);
  if constexpr (kAct == 1) y = round_bf16(gelu_tanh_<true>(y));
  if (has_res) y = round_bf16(y + res);
  return bf16_of_rounded(y);
}
// GeGLU (kAct == 2): gate and value = round(round(sum) + bias) - the contraction and the bias add
// are two tensor operations in the reference (torch/layers.py:700-703, torch/modules.py:749-751).
__device__ __forceinline__ float geglu_operand(float sum, float bias) {
  return round_bf16(round_bf16(sum) + bias);
}
__device__ __forceinline__ __nv_bfloat16 geglu_out(float gate, float value) {
  return bf16_of_rounded(round_bf16(round_bf16(gelu_tanh_<true>(gate)) * value));
}

struct SmallArgs {
  int M, m_pad, N, n_split;          // rows of x (and padded), features in all / in the first matrix
  int k_blocks, kb_per_split, splits;
  int n_stages, tmem_cols;
  int rows_per_rank, row_stride;     // rows of x a CTA of the cluster finishes; their pitch in the buffer
  int buf_off;                       // exchange buffer: behind the ring, or 0 = over the idle ring
  int bar_off;                       // barriers, TMEM address and abort flag behind ring and buffer
};

template <int kAct>
__global__ void __launch_bounds__(kThreadsS, 2)
gemm_small_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  const __grid_constant__ CUtensorMap map_w2, const __nv_bfloat16* __restrict__ bias,
                  const __nv_bfloat16* __restrict__ bias2, const __nv_bfloat16* __restrict__ residual,
                  const SmallArgs a, __nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ out2,
                  int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar0 = s_base + a.bar_off;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kMaxStagesS + s); };
  const uint32_t bar_acc = bar0 + 8u * (2 * kMaxStagesS);
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + a.bar_off + kOffTmemS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + a.bar_off + kOffAbortS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = a.M, m_pad = a.m_pad, N = a.N, splits = a.splits, n_stages = a.n_stages;
  const int n_tile = blockIdx.x;
  const int split = splits > 1 ? (int)cluster_rank() : 0;   // cluster = (1, splits, 1)
  const int n0 = n_tile * SN;
  // which of the two weight matrices this tile belongs to (n_split == N: only the first)
  const bool second = n0 >= a.n_split;
  const int lc0 = second ? n0 - a.n_split : n0;           // first feature within that matrix
  const int n_cols = second ? N - a.n_split : a.n_split;  // its feature count = its output's row length
  const __nv_bfloat16* tile_bias = second ? bias2 : bias;
  __nv_bfloat16* tile_out = second ? out2 : out;
  const int kb0 = split * a.kb_per_split;
  const int kb1 = min(kb0 + a.kb_per_split, a.k_blocks);
  const int n_kb = kb1 - kb0;
  const uint32_t stage_bytes = kWTile + static_cast<uint32_t>(m_pad) * SK * 2;   // [W 128 x 64][x m_pad x 64]
  const int pre = min(n_kb, n_stages);
  const bool own_buffer = a.buf_off != 0;       // the exchange buffer does not overlap the ring

  if (warp == kEpiS && lane == 0) {
    *s_abort = 0;
    for (int s = 0; s < kMaxStagesS; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    mbar_init(bar_acc, 1);
    mbar_fence_init();
    // the weights do not depend on the kernel before this one: their first stages are on their
    // way before anything else happens
    const CUtensorMap* mw = second ? &map_w2 : &map_w;
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(bar_full(i), stage_bytes);
      tma_load_2d(s_base + i * stage_bytes, mw, (kb0 + i) * SK, lc0, bar_full(i));
    }
  }
  if (warp == kEpiS + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(bar0 + kOffTmemS), "r"(a.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  // first cluster barrier: "this CTA runs, and its exchange buffer may be written".  With a buffer
  // of its own that holds from the start; over the ring it holds once the last MMA has read the ring.
  if (splits > 1 && own_buffer) cluster_arrive();
  grid_launch_dependents();
  grid_dependency_wait();

  if (warp == kEpiS) {
    // ------------------------------ TMA producer --------------------------------------------------
    if (lane == 0) {
      const CUtensorMap* mw = second ? &map_w2 : &map_w;
      for (int i = 0; i < pre; ++i)
        tma_load_2d(s_base + i * stage_bytes + kWTile, &map_x, (kb0 + i) * SK, 0, bar_full(i));
      bool ok = true;
      for (int i = pre; i < n_kb && ok; ++i) {
        const int s = i % n_stages;
        ok = mbar_wait(bar_empty(s), ((i / n_stages) & 1) ^ 1, s_abort);
        if (!ok) break;
        const uint32_t st = s_base + s * stage_bytes;
        mbar_expect_tx(bar_full(s), stage_bytes);
        tma_load_2d(st, mw, (kb0 + i) * SK, lc0, bar_full(s));
        tma_load_2d(st + kWTile, &map_x, (kb0 + i) * SK, 0, bar_full(s));
      }
    }
    __syncwarp();
  } else if (warp == kEpiS + 1) {
    // ------------------------------ MMA issue -----------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = tc_idesc_bf16(SN, m_pad);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % n_stages;
        ok = mbar_wait(bar_full(s), (i / n_stages) & 1, s_abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t w0 = s_base + s * stage_bytes, x0 = w0 + kWTile;
#pragma unroll
        for (int ks = 0; ks < SK / 16; ++ks)
          tc_mma_bf16(tmem_base, smem_desc_sw128(w0 + ks * 32), smem_desc_sw128(x0 + ks * 32), idesc,
                      (i | ks) != 0 ? 1u : 0u);
        tc_commit(bar_empty(s));
      }
      if (ok) tc_commit(bar_acc);
    }
    __syncwarp();
  }

  // ------------------------------ epilogue (warps 0-7) and the cluster exchange ------------------
  // a lane is a feature, an accumulator column a row of x; from 64 columns on, warps 4-7 take the
  // upper half of the columns
  const bool epi = warp < kEpiS;
  const int quarter = warp & 3, ch = warp >> 2;
  const int f = quarter * 32 + lane;                // feature within the tile
  const bool two_halves = m_pad >= 64;
  const int cols = two_halves ? m_pad / 2 : m_pad;
  const int col0 = two_halves ? ch * cols : 0;
  const bool warp_active = epi && (two_halves || ch == 0) && col0 < M;
  const bool f_ok = lc0 + f < n_cols;
  bool ok = true;
  if (epi || (splits > 1 && !own_buffer)) {
    if (lane == 0 || epi) ok = mbar_wait(bar_acc, 0, s_abort);
    __syncwarp();
    tc_fence_after();
  }
  const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);

  if (splits > 1) {
    // exchange buffer of a CTA: [source rank][feature 0..127][row_stride floats], the rows being the
    // rows_per_rank rows of x this CTA finishes.  rows_per_rank is a multiple of 4 and row_stride
    // an odd multiple of 4, so that 16-byte accesses of consecutive features fall on distinct banks.
    const int rpr = a.rows_per_rank, stride = a.row_stride;
    const uint32_t buf = s_base + (own_buffer ? a.buf_off : 0);
    if (!own_buffer) cluster_arrive();          // this CTA's ring is idle: every MMA has completed
    cluster_wait();                             // all peers run and their buffers may be written
    if (warp_active) {
      // my partial sums of row m go to the CTA that finishes row m, four rows per store
      const uint32_t my_slot = buf + static_cast<uint32_t>((split * SN + f) * stride) * 4;
      // each rank starts at another chunk of rows, so that at any time the CTAs of the cluster
      // write to different peers instead of all to the same one
      const int n_chunks = cols / 16;
      const int first = ((split + 1) * n_chunks / splits) % n_chunks;
#pragma unroll 2
      for (int k = 0; k < n_chunks; ++k) {
        uint32_t acc[16];
        const int c = ((first + k) % n_chunks) * 16;
        if (col0 + c >= M) continue;            // only padding in this chunk
        tc_ld_32x16(t_row + col0 + c, acc);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          const int m = col0 + c + j;
          if (m < M) {                          // m is a multiple of 4 and so is rpr: one rank
            const int d = m / rpr, lm = m - d * rpr;
            asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};"
                         :: "r"(peer_smem(my_slot, d) + lm * 4), "r"(acc[j]), "r"(acc[j + 1]),
                            "r"(acc[j + 2]), "r"(acc[j + 3]) : "memory");
          }
        }
      }
    }
    cluster_arrive();
    cluster_wait();
    // the rows [split * rpr, split * rpr + rpr) of x are mine to finish: slices added in rank order
    if (epi && ok) {
      const float* sums = reinterpret_cast<const float*>(smem + (own_buffer ? a.buf_off : 0));
      const int m_base = split * rpr;
      if constexpr (kAct == 2) {
        const int g = threadIdx.x & 63;           // output feature within the group of 64
        const float bg = bf16_value(bias[n0 + g]), bv = bf16_value(bias[n0 + 64 + g]);
        for (int lm = (threadIdx.x >> 6) * 4; lm < rpr && m_base + lm < M; lm += (kEpiS / 2) * 4) {
          float4 sg = make_float4(0.f, 0.f, 0.f, 0.f), sv = sg;
          for (int s = 0; s < splits; ++s) {
            const float4 pg = *reinterpret_cast<const float4*>(sums + (s * SN + g) * stride + lm);
            const float4 pv = *reinterpret_cast<const float4*>(sums + (s * SN + 64 + g) * stride + lm);
            sg.x += pg.x; sg.y += pg.y; sg.z += pg.z; sg.w += pg.w;
            sv.x += pv.x; sv.y += pv.y; sv.z += pv.z; sv.w += pv.w;
          }
          const float gs[4] = {sg.x, sg.y, sg.z, sg.w}, vs[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int m = m_base + lm + j;
            if (m < M)
              out[(int64_t)m * (N / 2) + n_tile * 64 + g] =
                  geglu_out(geglu_operand(gs[j], bg), geglu_operand(vs[j], bv));
          }
        }
      } else {
        const int ff = threadIdx.x & 127;
        if (lc0 + ff < n_cols) {
          const float b = tile_bias != nullptr ? bf16_value(tile_bias[lc0 + ff]) : 0.0f;
          const bool has_res = residual != nullptr;
          for (int lm = (threadIdx.x >> 7) * 4; lm < rpr && m_base + lm < M; lm += (kEpiS / 4) * 4) {
            float rs[4] = {0.f, 0.f, 0.f, 0.f};
            if (has_res) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int m = m_base + lm + j;
                if (m < M) rs[j] = bf16_value(residual[(int64_t)m * n_cols + lc0 + ff]);
              }
            }
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < splits; ++s) {
              const float4 p = *reinterpret_cast<const float4*>(sums + (s * SN + ff) * stride + lm);
              sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
            }
            const float vs[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int m = m_base + lm + j;
              if (m < M) tile_out[(int64_t)m * n_cols + lc0 + ff] = finish1<kAct>(vs[j], b, has_res, rs[j]);
            }
          }
        }
      }
    }
  } else if (kAct == 2) {
    // a single K slice, GeGLU: the tile is one group of the packed up-projection, features 0-63
    // gates, 64-127 the values of the same outputs.  The value warps leave their operands in the
    // (idle) ring, the gate warps pick them up.
    if (epi) {
      __nv_bfloat16* s_val = reinterpret_cast<__nv_bfloat16*>(smem);   // [m][64]
      const float b = bf16_value(bias[n0 + f]);
      if (warp_active && quarter >= 2) {
#pragma unroll 1
        for (int c = 0; c < cols; c += 16) {
          uint32_t acc[16];
          tc_ld_32x16(t_row + col0 + c, acc);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = col0 + c + j;
            if (m < M) s_val[m * 64 + f - 64] = bf16_of_rounded(geglu_operand(__uint_as_float(acc[j]), b));
          }
        }
      }
      named_bar_sync(1, kEpiS * 32);
      if (warp_active && quarter < 2 && ok) {
#pragma unroll 1
        for (int c = 0; c < cols; c += 16) {
          uint32_t acc[16];
          tc_ld_32x16(t_row + col0 + c, acc);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = col0 + c + j;
            if (m < M)
              out[(int64_t)m * (N / 2) + n_tile * 64 + f] =
                  geglu_out(geglu_operand(__uint_as_float(acc[j]), b), bf16_value(s_val[m * 64 + f]));
          }
        }
      }
    }
  } else if (warp_active) {
    // a single K slice: the output straight from tensor memory
    const float b = (tile_bias != nullptr && f_ok) ? bf16_value(tile_bias[lc0 + f]) : 0.0f;
    const bool has_res = residual != nullptr;
#pragma unroll 2
    for (int c = 0; c < cols; c += 16) {
      uint32_t acc[16];
      tc_ld_32x16(t_row + col0 + c, acc);
      tc_wait_ld();
      if (ok && f_ok) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = col0 + c + j;
          if (m < M) {
            if constexpr (kAct != 2) {
              const int64_t o = (int64_t)m * n_cols + lc0 + f;
              const float r = has_res ? bf16_value(residual[o]) : 0.0f;
              tile_out[o] = finish1<kAct>(__uint_as_float(acc[j]), b, has_res, r);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *s_abort && status != nullptr) atomicExch(status, kStatusTimeout);
  if (warp == kEpiS + 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(a.tmem_cols)
                 : "memory");
  }
}

template <int kAct>
cudaError_t launch_small(const cudaLaunchConfig_t& cfg, const CUtensorMap& mx, const CUtensorMap& mw,
                         const CUtensorMap& mw2, const void* bias, const void* bias2,
                         const void* residual, const SmallArgs& a, void* out, void* out2, int* status) {
  using T_ = __nv_bfloat16;
  return cudaLaunchKernelEx(&cfg, gemm_small_kernel<kAct>, mx, mw, mw2, (const T_*)bias, (const T_*)bias2,
                            (const T_*)residual, a, (T_*)out, (T_*)out2, status);
}

// How many clusters of `c` CTAs of this kernel the current device runs at once with `smem` bytes of
// dynamic shared memory per CTA (clusters do not span GPCs, so this is less than SMs / c); cached
// per device for the two sizes the launcher uses.
int max_active_clusters(int c, int smem, int which) {
  static std::mutex mu;
  static int cache[64][2][kMaxClusterS + 1] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev][which][c] == 0) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)c;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, (unsigned)c);
    cfg.blockDim = dim3(kThreadsS);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_small_kernel<0>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    cache[dev][which][c] = n > 0 ? n : -1;
  }
  return cache[dev][which][c] > 0 ? cache[dev][which][c] : 0;
}

// Shared-memory plan for `budget` bytes of ring + exchange buffer: the buffer behind the ring if
// that leaves the ring enough stages, else over the ring (written once the ring is idle).
bool plan_smem(SmallArgs* a, int budget, int stage, int buf_bytes, int min_stages) {
  const int most = a->kb_per_split < kMaxStagesS ? a->kb_per_split : kMaxStagesS;
  const int need = min_stages < most ? min_stages : most;
  int ns = (budget - buf_bytes) / stage;
  if (ns >= need) {
    a->n_stages = ns < most ? ns : most;
    a->buf_off = buf_bytes > 0 ? a->n_stages * stage : 0;
    a->bar_off = a->n_stages * stage + buf_bytes;
    return true;
  }
  ns = budget / stage;
  if (ns < need || buf_bytes > budget) return false;
  a->n_stages = ns < most ? ns : most;
  a->buf_off = 0;
  a->bar_off = a->n_stages * stage > buf_bytes ? a->n_stages * stage : buf_bytes;
  return true;
}

}  // namespace

bool dense_small_supported(int dtype, int64_t M, int64_t K, int64_t N) {
  return dtype == 1 && M >= 1 && M <= 256 && K >= 8 && N >= 8 && K % 8 == 0 && N % 8 == 0 &&
         K < (1 << 30) && N < (1 << 30);
}

cudaError_t launch_dense_small(const void* x, const void* w, const void* bias, const void* w2,
                               const void* bias2, const void* residual, int64_t M, int K, int N,
                               int N2, int act, void* out, void* out2, int* status, cudaStream_t s) {
  const bool pair = w2 != nullptr;
  if (pair && (N % SN != 0 || act == 2 || residual != nullptr || out2 == nullptr)) return cudaErrorInvalidValue;
  if (act == 2 && (residual != nullptr || N % SN != 0 || bias == nullptr)) return cudaErrorInvalidValue;
  static PerDeviceOnce once;
  int num_sms = 0;
  cudaError_t e0 = once.run([] {
    cudaError_t e = cudaFuncSetAttribute(gemm_small_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDataS + kTailS);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(gemm_small_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDataS + kTailS);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_small_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDataS + kTailS);
  }, &num_sms);
  if (e0 != cudaSuccess) return e0;

  SmallArgs a;
  a.M = (int)M;
  // the narrow operand's row count: a multiple of 16, of 32 from 64 on (the epilogue halves it)
  a.m_pad = M <= 48 ? (int)((M + 15) / 16) * 16 : (int)((M + 31) / 32) * 32;
  a.tmem_cols = 32;
  while (a.tmem_cols < a.m_pad) a.tmem_cols *= 2;
  a.N = N + (pair ? N2 : 0);
  a.n_split = N;
  const int n_tiles = (a.N + SN - 1) / SN;
  a.k_blocks = (K + SK - 1) / SK;
  const int stage = kWTile + a.m_pad * SK * 2;
  // Up to 128 rows the CTA is sized so that two fit an SM: the CTAs of the next kernel in the
  // stream (launched as its programmatic dependent) then fetch their weights while this one
  // exchanges and finishes.  K slices = the largest cluster whose clusters all run at once, one
  // CTA per SM.
  // (Not when a CTA streams more K blocks than the full ring holds: such a call is long enough to
  // want every stage for itself.)
  bool planned = false;
  const bool long_k = (a.k_blocks + kMaxClusterS - 1) / kMaxClusterS > kMaxStagesS ||
                      n_tiles * 2 > num_sms;
  for (int half = (a.m_pad <= 128 && !long_k) ? 1 : 0; half >= 0 && !planned; --half) {
    const int budget = half ? kDataHalfS : kDataS;
    int c = a.k_blocks < kMaxClusterS ? a.k_blocks : kMaxClusterS;
    while (c > 1 && (n_tiles * c > num_sms || max_active_clusters(c, budget + kTailS, half) < n_tiles)) --c;
    a.kb_per_split = (a.k_blocks + c - 1) / c;
    a.splits = (a.k_blocks + a.kb_per_split - 1) / a.kb_per_split;
    a.rows_per_rank = ((int)((M + a.splits - 1) / a.splits) + 3) & ~3;
    a.row_stride = (a.rows_per_rank / 4) % 2 == 1 ? a.rows_per_rank : a.rows_per_rank + 4;
    const int buf_bytes = a.splits > 1 ? a.splits * SN * a.row_stride * 4 : 0;
    planned = plan_smem(&a, budget, stage, buf_bytes, half ? 2 : 1);
  }
  if (!planned) return cudaErrorInvalidValue;
  const int smem_bytes = a.bar_off + kTailS;

  CUtensorMap map_x, map_w, map_w2;
  if (!tensor_map_2d(&map_x, x, (uint64_t)M, (uint64_t)K, (uint32_t)a.m_pad, SK, true) ||
      !tensor_map_2d(&map_w, w, (uint64_t)N, (uint64_t)K, SN, SK, true))
    return cudaErrorInvalidValue;
  if (!pair) map_w2 = map_w;
  else if (!tensor_map_2d(&map_w2, w2, (uint64_t)N2, (uint64_t)K, SN, SK, true)) return cudaErrorInvalidValue;

  // may start while the kernel before it in the stream drains (see grid_dependency_wait)
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;       // the K slices of a feature tile
  attr[1].val.clusterDim.x = 1;
  attr[1].val.clusterDim.y = (unsigned)a.splits;
  attr[1].val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)n_tiles, (unsigned)a.splits);
  cfg.blockDim = dim3(kThreadsS);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = a.splits > 1 ? 2 : 1;
  cudaError_t e;
  if (act == 2) e = launch_small<2>(cfg, map_x, map_w, map_w2, bias, bias2, residual, a, out, out2, status);
  else if (act == 1) e = launch_small<1>(cfg, map_x, map_w, map_w2, bias, bias2, residual, a, out, out2, status);
  else e = launch_small<0>(cfg, map_x, map_w, map_w2, bias, bias2, residual, a, out, out2, status);
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace rgk
