// Dense projection out = x W^T + b (torch.nn.Linear as RecurrentBlock uses it, recurrentgemma
// torch/modules.py:531-548, 627-631, 647) on the 5th-generation tensor cores, bfloat16 in and out,
// float32 accumulation, optional gelu_tanh epilogue (the y branch, torch/modules.py:628).
//
// x [M, K] and W [N, K] are both K-contiguous, i.e. K-major operands as they are: TMA brings
// 128 x 64 (x) and 256 x 64 (W) boxes with the 128-byte swizzle into a 4-stage ring, a single
// thread issues tcgen05.mma.cta_group::1.kind::f16 (M 128, N 256, K 16) into one of two TMEM
// accumulators, and 16 epilogue warps drain the other: tcgen05.ld, + bias in float32, one rounding
// to bfloat16 (then gelu and a second rounding if asked, as torch does for a separate gelu op),
// a 32 x 32 transposition through shared memory and 64-byte-contiguous stores.  Persistent CTAs
// walk the output tiles n-fastest so that the CTAs running together share x rows and all of W in L2.
//
// Every mbarrier wait is bounded; on expiry WsHeader::status (if given) is raised and the CTA leaves.
#include <cuda.h>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tc_common.cuh"

namespace rgk {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, kStages = 4;
constexpr int kABytes = BM * BK * 2;             // 16 KiB
constexpr int kBBytes = BN * BK * 2;             // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;   // 48 KiB
constexpr int kEpi = 16;
constexpr int kThreadsG = (kEpi + 2) * 32;
constexpr int kOffRing = 0;
constexpr int kOffStageOut = kStages * kStageBytes;              // 196608: per-warp 2 KiB staging
constexpr int kOffBarG = kOffStageOut + kEpi * 2048;             // full[4] empty[4] acc_full[2] acc_empty[2]
constexpr int kOffTmemG = kOffBarG + (2 * kStages + 4) * 8;
constexpr int kOffAbortG = kOffTmemG + 4;
constexpr int kSmemG = kOffAbortG + 4 + 1024;
static_assert(kSmemG <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");
constexpr uint32_t kIdescG = tc_idesc_bf16(BM, BN);

// kMode 0: bias only; 1: gelu_tanh of the rounded result; 2: + residual (rounded again);
// 3: GeGLU - W holds, per group of 128 rows, 64 gate rows then the 64 value rows of the same
//    features (see pack_mlp_up_kernel); out [M, N/2] = gelu_tanh(gate) * value, where gate and
//    value are round(round(acc) + bias): the contraction and the bias add are two tensor operations
//    in the reference (torch/layers.py:700-703, torch/modules.py:749-751);
// 4: logits soft cap - round(tanh(round(round(acc) / cap)) * cap), the three tensor operations of
//    torch/griffin.py:183-185 after the contraction of torch/modules.py:1003.
template <int kMode>
__global__ void __launch_bounds__(kThreadsG, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ residual,
               int64_t M, int N, int K, int m_tiles,
               int n_tiles, __nv_bfloat16* __restrict__ out, int* status, float cap) {
  extern __shared__ uint8_t smem_raw[];
  // aligned by an offset into the shared array, so that the address space stays known to the
  // compiler (shared-memory load/store instructions instead of generic ones)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar0 = s_base + kOffBarG;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto bar_acc_full = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
  auto bar_acc_empty = [&](int s) { return bar0 + 8u * (2 * kStages + 2 + s); };
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + kOffTmemG);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffAbortG);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (K + BK - 1) / BK;
  const int total_tiles = m_tiles * n_tiles;
  const int n_my = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(bar_acc_full(s), 1); mbar_init(bar_acc_empty(s), kEpi / 2); }
    mbar_fence_init();
  }
  if (warp == kEpi + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(s_base + kOffTmemG), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == kEpi) {
    // ------------------------------ TMA producer --------------------------------------------------
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int t = 0; t < n_my && ok; ++t) {
        const int tile = blockIdx.x + t * gridDim.x;
        const int m0 = (tile / n_tiles) * BM, n0 = (tile % n_tiles) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          ok = mbar_wait(bar_empty(s), ((it / kStages) & 1) ^ 1, s_abort);
          if (!ok) break;
          mbar_expect_tx(bar_full(s), kStageBytes);
          tma_load_2d(s_base + kOffRing + s * kStageBytes, &map_x, kb * BK, m0, bar_full(s));
          tma_load_2d(s_base + kOffRing + s * kStageBytes + kABytes, &map_w, kb * BK, n0, bar_full(s));
        }
      }
    }
  } else if (warp == kEpi + 1) {
    // ------------------------------ MMA issue -----------------------------------------------------
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int t = 0; t < n_my && ok; ++t) {
        const int as = t & 1;
        ok = mbar_wait(bar_acc_empty(as), ((t >> 1) & 1) ^ 1, s_abort);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          ok = mbar_wait(bar_full(s), (it / kStages) & 1, s_abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a0 = s_base + kOffRing + s * kStageBytes, b0 = a0 + kABytes;
#pragma unroll
          for (int ks = 0; ks < BK / 16; ++ks)
            tc_mma_bf16(tmem_base + as * BN, smem_desc_sw128(a0 + ks * 32),
                        smem_desc_sw128(b0 + ks * 32), kIdescG, (kb | ks) != 0 ? 1u : 0u);
          tc_commit(bar_empty(s));
        }
        if (ok) tc_commit(bar_acc_full(as));
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------------------------------
    const int as = warp >> 3;                // accumulator = tile parity
    const int lane_base = (warp & 3) * 32;   // TMEM lanes this warp may read
    const int col_half = (warp >> 2) & 1;    // which 128 of the tile's 256 columns
    uint8_t* stage = smem + kOffStageOut + warp * 2048;
    bool ok = true;
    for (int t = as; t < n_my && ok; t += 2) {
      const int tile = blockIdx.x + t * gridDim.x;
      const int64_t m0 = (int64_t)(tile / n_tiles) * BM;
      const int n0 = (tile % n_tiles) * BN + col_half * 128;
      ok = mbar_wait(bar_acc_full(as), (t >> 1) & 1, s_abort);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + as * BN +
                             col_half * 128;
      if constexpr (kMode == 3) {
        // this warp's 128 accumulator columns are one group: gate columns 0-63, value columns 64-127
        const int n_out = N / 2;
        const int oc0 = n0 / 2;                // first output feature of the group
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {       // 32 features at a time
          uint4 ov[4];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {     // 16 features: bounded register use
            uint32_t ag[16], av[16];
            tc_ld_32x16(t_row + cc * 32 + hf * 16, ag);
            tc_ld_32x16(t_row + 64 + cc * 32 + hf * 16, av);
            const int nb = n0 + cc * 32 + hf * 16;
            uint4 bg[2], bvv[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              bg[j] = *reinterpret_cast<const uint4*>(bias + nb + 8 * j);
              bvv[j] = *reinterpret_cast<const uint4*>(bias + nb + 64 + 8 * j);
            }
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const uint32_t bgp[4] = {bg[j].x, bg[j].y, bg[j].z, bg[j].w};
              const uint32_t bvp[4] = {bvv[j].x, bvv[j].y, bvv[j].z, bvv[j].w};
              uint32_t o[4];
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                const int n = j * 8 + p * 2;
                const uint32_t g2 = badd2(pack_bf16x2(__uint_as_float(ag[n]), __uint_as_float(ag[n + 1])), bgp[p]);
                const uint32_t v2 = badd2(pack_bf16x2(__uint_as_float(av[n]), __uint_as_float(av[n + 1])), bvp[p]);
                const uint32_t a2 = pack_bf16x2(gelu_tanh_<true>(bf16_lo(g2)), gelu_tanh_<true>(bf16_hi(g2)));
                o[p] = bmul2(a2, v2);
              }
              ov[hf * 2 + j] = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(stage + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = ov[j];
          __syncwarp();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int r = (lane >> 2) + 8 * k, piece = lane & 3;
            const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 64 + ((piece ^ ((r >> 1) & 3)) << 4));
            const int64_t grow = m0 + lane_base + r;
            const int gcol = oc0 + cc * 32 + piece * 8;
            if (grow < M && gcol < n_out) *reinterpret_cast<uint4*>(out + grow * n_out + gcol) = v;
          }
          __syncwarp();
        }
      } else {
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t acc[32];
        tc_ld_32x32(t_row + cc * 32, acc);
        const int nc = n0 + cc * 32;         // first output column of this chunk
        // the residual pieces this thread will add after the transposition: in flight during the
        // epilogue arithmetic
        uint4 rv[4];
        if constexpr (kMode == 2) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int64_t grow = m0 + lane_base + (lane >> 2) + 8 * k;
            const int gcol = nc + (lane & 3) * 8;
            rv[k] = (grow < M && gcol < N) ? ld_stream(residual + grow * N + gcol)
                                           : make_uint4(0u, 0u, 0u, 0u);
          }
        }
        float bv[32];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          uint32_t b2 = 0u;
          if (bias != nullptr && nc + j < N) b2 = *reinterpret_cast<const uint32_t*>(bias + nc + j);
          bv[j] = bf16_lo(b2); bv[j + 1] = bf16_hi(b2);
        }
        tc_wait_ld();
        uint4 ov[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t o[4];
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const int n = j * 8 + p * 2;
            float v0 = __uint_as_float(acc[n]) + bv[n], v1 = __uint_as_float(acc[n + 1]) + bv[n + 1];
            uint32_t pk = pack_bf16x2(v0, v1);
            if constexpr (kMode == 1) pk = pack_bf16x2(gelu_tanh_<true>(bf16_lo(pk)), gelu_tanh_<true>(bf16_hi(pk)));
            if constexpr (kMode == 4) {
              uint32_t t = pack_bf16x2(__fdiv_rn(bf16_lo(pk), cap), __fdiv_rn(bf16_hi(pk), cap));
              t = pack_bf16x2(tanhf(bf16_lo(t)), tanhf(bf16_hi(t)));
              pk = pack_bf16x2(bf16_lo(t) * cap, bf16_hi(t) * cap);
            }
            o[p] = pk;
          }
          ov[j] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        // 32 x 32 transposition through the warp's staging buffer (see gates_tc.cu), then stores of
        // 8 rows x 64 contiguous bytes per instruction.
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(stage + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = ov[j];
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int r = (lane >> 2) + 8 * k, piece = lane & 3;
          uint4 v = *reinterpret_cast<const uint4*>(stage + r * 64 + ((piece ^ ((r >> 1) & 3)) << 4));
          const int64_t grow = m0 + lane_base + r;
          const int gcol = nc + piece * 8;
          if (grow < M && gcol < N) {
            if constexpr (kMode == 2) {
              // the residual stream joins here: round(round(acc + bias) + residual), the two tensor
              // operations of the reference (torch/modules.py:899-902)
              v = make_uint4(badd2(v.x, rv[k].x), badd2(v.y, rv[k].y), badd2(v.z, rv[k].z),
                             badd2(v.w, rv[k].w));
            }
            *reinterpret_cast<uint4*>(out + grow * N + gcol) = v;
          }
        }
        __syncwarp();
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(as));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *s_abort && status != nullptr) atomicExch(status, kStatusTimeout);
  if (warp == kEpi + 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512)
                 : "memory");
  }
}

// ffw_up of the MLP block: w [2, D, X] (in, out) and b [2, X] into the K-major, gate/value
// interleaved layout of mode 3: packed row g*128 + c*64 + i = column (feature) g*64 + i of w[c].
__global__ void pack_mlp_up_kernel(const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                                   int D, int X, __nv_bfloat16* __restrict__ packed_w,
                                   __nv_bfloat16* __restrict__ packed_b) {
  __shared__ __nv_bfloat16 tile[32][33];
  // grid: (D / 32 rounded up, X / 32, 2); block 32 x 8
  const int c = blockIdx.z, k0 = blockIdx.x * 32, f0 = blockIdx.y * 32;
  const __nv_bfloat16* src = w + (int64_t)c * D * X;
  for (int r = threadIdx.y; r < 32; r += 8) {                      // r walks k, x walks features
    const int k = k0 + r, f = f0 + threadIdx.x;
    tile[r][threadIdx.x] = (k < D && f < X) ? src[(int64_t)k * X + f] : __float2bfloat16(0.0f);
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += 8) {                      // r walks features, x walks k
    const int f = f0 + r, k = k0 + threadIdx.x;
    if (f < X && k < D) {
      const int64_t row = (int64_t)(f / 64) * 128 + c * 64 + (f % 64);
      packed_w[row * D + k] = tile[threadIdx.x][r];
      if (k == 0) packed_b[row] = b[(int64_t)c * X + f];
    }
  }
}



}  // namespace

bool dense_tc_supported(int dtype, int64_t M, int64_t K, int64_t N) {
  return dtype == 1 && M >= 1 && M < ((int64_t)1 << 31) && K >= 8 && K % 8 == 0 && N >= 8 &&
         N % 8 == 0 && K < (1 << 24) && N < (1 << 24);
}

cudaError_t launch_dense_tc(const void* x, const void* w, const void* bias, const void* residual,
                            int64_t M, int K, int N, int gelu, void* out, int* status,
                            cudaStream_t s, float cap) {
  if (M == 0) return cudaSuccess;
  CUtensorMap map_x, map_w;
  if (!tensor_map_2d(&map_x, x, (uint64_t)M, (uint64_t)K, BM, BK, true) ||
      !tensor_map_2d(&map_w, w, (uint64_t)N, (uint64_t)K, BN, BK, true))
    return cudaErrorInvalidValue;
  static PerDeviceOnce once;
  int num_sms = 0;
  cudaError_t e0 = once.run([] {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemm_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemG)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemG)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(gemm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemG)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(gemm_tc_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemG)) != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemG);
  }, &num_sms);
  if (e0 != cudaSuccess) return e0;
  const int m_tiles = (int)((M + BM - 1) / BM), n_tiles = (N + BN - 1) / BN;
  const int total = m_tiles * n_tiles;
  const int grid = total < num_sms ? total : num_sms;
  using T_ = __nv_bfloat16;
  if ((gelu != 0) + (residual != nullptr) > 1) return cudaErrorInvalidValue;
#define RGK_GEMM(MODE)                                                                          \
  gemm_tc_kernel<MODE><<<grid, kThreadsG, kSmemG, s>>>(map_x, map_w, (const T_*)bias,           \
                                                       (const T_*)residual, M, N, K, m_tiles,   \
                                                       n_tiles, (T_*)out, status, cap)
  if (cap != 0.0f && (gelu != 0 || residual != nullptr || bias != nullptr)) return cudaErrorInvalidValue;
  if (cap != 0.0f) RGK_GEMM(4);
  else if (gelu == 2) RGK_GEMM(3); else if (gelu) RGK_GEMM(1); else if (residual) RGK_GEMM(2); else RGK_GEMM(0);
#undef RGK_GEMM
  return cudaGetLastError();
}

cudaError_t launch_pack_mlp_up(const void* w, const void* b, int D, int X, void* packed_w,
                               void* packed_b, cudaStream_t s) {
  using T_ = __nv_bfloat16;
  const dim3 grid((unsigned)((D + 31) / 32), (unsigned)((X + 31) / 32), 2), block(32, 8);
  pack_mlp_up_kernel<<<grid, block, 0, s>>>((const T_*)w, (const T_*)b, D, X, (T_*)packed_w,
                                           (T_*)packed_b);
  return cudaGetLastError();
}

}  // namespace rgk
