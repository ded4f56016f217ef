// Block-diagonal gate projections of the RG-LRU in float32 on the 5th-generation tensor cores,
// fused with the gate arithmetic (recurrentgemma torch/layers.py:127-137, 338-353), for heads of
// width 256.
//
// The tensor cores have no float32 multiply; kind::tf32 reads the upper 19 bits of a float32
// (10 mantissa bits).  A float32 product is recovered to well below the 1e-5 parity bar from three
// TF32 products with a float32 accumulator ("3xTF32"):
//     x w  ~  x_hi w_hi + x_lo w_hi + x_hi w_lo,     v_hi = v with the low 13 mantissa bits cleared,
//                                                    v_lo = v - v_hi (exact in float32)
// (the dropped x_lo w_lo term is below 2^-22 of the product).  The activations are split on chip, per
// K-slice, by the warps that later run the epilogue (hi written back over the slice the copy engine
// delivered, lo beside it); the weights are split by a packing kernel into two K-major arrays.
//
// One CTA per (128-token tile, head, channel half): N = 256 accumulator columns = the 128 x-gate and
// the 128 a-gate outputs of the half's channels, so that an epilogue thread finds both gates of a
// channel in its own TMEM lane.  K = 256 arrives in sixteen slices of 16 (64-byte rows, 64-byte
// swizzle) through a four-stage ring: activations 8 KiB, their low part 8 KiB (written by the
// helper warps), weights hi and lo 16 KiB each - the per-slice hand-offs (copy engine -> split ->
// tensor core -> release) of a CTA are serial, so more and smaller stages in flight hide them.  A single thread issues three
// tcgen05.mma.cta_group::1.kind::tf32 (M 128, N 256, K 8) per K step.  The epilogue (16 warps: TMEM
// lane quarter x 32-channel chunk) reads the accumulators, applies the float32-accurate gate
// arithmetic and writes a and the normalised input for the scan kernel.
//
// Every mbarrier wait is bounded; on expiry WsHeader::status is raised and the CTA leaves.
#include <cuda.h>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tc_common.cuh"

namespace rgk {
namespace {

constexpr int kHW = 256;                 // head width = K
constexpr int kTM = 128;                 // tokens per tile (MMA M)
constexpr int kTN = 256;                 // accumulator columns: 128 x-gate + 128 a-gate
constexpr int kHalf = 128;               // channels per CTA
constexpr int kKS = 16;                  // K per slice: 16 float32 = 64 bytes (64-byte swizzle); 32 also works
constexpr int kSlices = kHW / kKS;
constexpr int kStages = 64 / kKS;        // 4 stages of 48 KiB, or 2 of 96 KiB
constexpr int kABytes = kTM * kKS * 4;
constexpr int kBBytes = kTN * kKS * 4;
constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;     // A, A_lo, B_hi, B_lo
constexpr bool kSw128 = kKS == 32;
__device__ __forceinline__ uint64_t tf32_desc(uint32_t addr) {
  return kSw128 ? smem_desc_sw128(addr) : smem_desc_sw64(addr);
}
constexpr int kEpi = 16;
constexpr int kThreadsF = (kEpi + 2) * 32;
constexpr int kOffSp = kStages * kStageBytes;               // float [3][128]: softplus(a_param), gate biases
constexpr int kOffBarF = kOffSp + 3 * kHalf * 4;                // full[2] lo_full[2] empty[2] acc_full
constexpr int kNumBarF = 3 * kStages + 1;
constexpr int kOffTmemF = kOffBarF + kNumBarF * 8;
constexpr int kOffAbortF = kOffTmemF + 4;
constexpr int kSmemF = kOffAbortF + 4 + 1024;
static_assert(kSmemF <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");

// Instruction descriptor of tcgen05.mma kind::tf32: D float32, A and B TF32, both K-major.
constexpr uint32_t tc_idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
constexpr uint32_t kIdescF = tc_idesc_tf32(kTM, kTN);

__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// v with the low 13 mantissa bits cleared (an exact TF32 value), and the rest of v (exact).
__device__ __forceinline__ float tf32_high_part(float v) {
  return __uint_as_float(__float_as_uint(v) & 0xffffe000u);
}
__device__ __forceinline__ float tf32_low_part(float v) { return v - tf32_high_part(v); }

__global__ void __launch_bounds__(kThreadsF, 1)
gates_tf32_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wh,
                  const __grid_constant__ CUtensorMap map_wl, const float* __restrict__ x,
                  const void* __restrict__ pos, int pos64, const float* __restrict__ a_param,
                  const float* __restrict__ bias_x, const float* __restrict__ bias_a, int64_t M,
                  int E, float* __restrict__ a_out, float* __restrict__ xn_out, WsHeader* hdr) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar0 = s_base + kOffBarF;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_lo = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto bar_empty = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
  const uint32_t bar_acc = bar0 + 8u * (3 * kStages);
  float* s_sp = reinterpret_cast<float*>(smem + kOffSp);
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + kOffTmemF);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffAbortF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, group = blockIdx.y;          // (head, half)
  const int head = group >> 1, half = group & 1;
  const int chan0 = head * kHW + half * kHalf;

  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_lo(s), kEpi);
      mbar_init(bar_empty(s), 1);
    }
    mbar_init(bar_acc, 1);
    mbar_fence_init();
  }
  if (warp == kEpi + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(s_base + kOffTmemF), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x < kHalf) {
    s_sp[threadIdx.x] = softplus_(a_param[chan0 + threadIdx.x]);
    s_sp[kHalf + threadIdx.x] = bias_x[chan0 + threadIdx.x];
    s_sp[2 * kHalf + threadIdx.x] = bias_a[chan0 + threadIdx.x];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == kEpi) {
    // ------------------------------ TMA producer --------------------------------------------------
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < kSlices && ok; ++kb) {
        const int s = kb % kStages;
        ok = mbar_wait(bar_empty(s), ((kb / kStages) & 1) ^ 1, s_abort);
        if (!ok) break;
        const uint32_t st = s_base + s * kStageBytes;
        mbar_expect_tx(bar_full(s), kABytes + 2 * kBBytes);
        tma_load_2d(st, &map_x, head * kHW + kb * kKS, tile * kTM, bar_full(s));
        tma_load_2d(st + 2 * kABytes, &map_wh, kb * kKS, group * kTN, bar_full(s));
        tma_load_2d(st + 2 * kABytes + kBBytes, &map_wl, kb * kKS, group * kTN, bar_full(s));
      }
    }
  } else if (warp == kEpi + 1) {
    // ------------------------------ MMA issue -----------------------------------------------------
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < kSlices && ok; ++kb) {
        const int s = kb % kStages;
        ok = mbar_wait(bar_full(s), (kb / kStages) & 1, s_abort);
        if (ok) ok = mbar_wait(bar_lo(s), (kb / kStages) & 1, s_abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_hi = s_base + s * kStageBytes, a_lo = a_hi + kABytes;
        const uint32_t b_hi = a_hi + 2 * kABytes, b_lo = b_hi + kBBytes;
#pragma unroll
        for (int ks = 0; ks < kKS / 8; ++ks) {
          const uint64_t dah = tf32_desc(a_hi + ks * 32), dal = tf32_desc(a_lo + ks * 32);
          const uint64_t dbh = tf32_desc(b_hi + ks * 32), dbl = tf32_desc(b_lo + ks * 32);
          tc_mma_tf32(tmem_base, dah, dbh, kIdescF, (kb | ks) != 0 ? 1u : 0u);
          tc_mma_tf32(tmem_base, dal, dbh, kIdescF, 1u);
          tc_mma_tf32(tmem_base, dah, dbl, kIdescF, 1u);
        }
        tc_commit(bar_empty(s));
      }
      if (ok) tc_commit(bar_acc);
    }
  } else {
    // ------------------------------ helper, then epilogue ------------------------------------------
    // During the main loop: the low parts of the activation slice (element-wise, so the swizzled
    // layout carries over address for address).  512 threads cover one 128-token slice.
    bool ok = true;
    for (int kb = 0; kb < kSlices && ok; ++kb) {
      const int s = kb % kStages;
      ok = mbar_wait(bar_full(s), (kb / kStages) & 1, s_abort);
      if (!ok) break;
      constexpr int kPer = kABytes / 16 / (kEpi * 32);          // 16-byte pieces per thread
      float4* src = reinterpret_cast<float4*>(smem + s * kStageBytes) + threadIdx.x * kPer;
      float4* dst = reinterpret_cast<float4*>(smem + s * kStageBytes + kABytes) + threadIdx.x * kPer;
#pragma unroll
      for (int i = 0; i < kPer; ++i) {
        const float4 v = src[i];
        dst[i] = make_float4(tf32_low_part(v.x), tf32_low_part(v.y), tf32_low_part(v.z),
                             tf32_low_part(v.w));
        // the high part is written back explicitly, so that the split does not depend on how the
        // tensor core narrows a float32 operand (an exact TF32 value passes unchanged either way)
        src[i] = make_float4(tf32_high_part(v.x), tf32_high_part(v.y), tf32_high_part(v.z),
                             tf32_high_part(v.w));
      }
      fence_proxy_async();                  // the tensor core reads this through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_lo(s));
    }
    // Epilogue: thread = token row of the warp's TMEM lane quarter, 32 channels of the half.
    // Global traffic goes through two per-warp 32 x 32 float32 blocks in the (now idle) ring, so that
    // a load or store instruction moves four rows x 128 contiguous bytes instead of 32 rows x 16
    // bytes: 16-byte piece j of row r sits at piece j ^ (r & 7), conflict-free both for the row
    // owner (lane = row) and for the copy pattern (8 lanes per row).
    const int lane_base = (warp & 3) * 32;
    const int cq = warp >> 2;                                // 32-channel chunk of the half
    const int64_t row0 = (int64_t)tile * kTM + lane_base;
    const int64_t row = row0 + lane;
    const bool is_reset = row < M && pos_is_zero(pos, pos64, row);
    const int e0 = chan0 + cq * 32;
    uint8_t* blk_a = smem + warp * 8192;                     // conv values in, a out
    uint8_t* blk_x = blk_a + 4096;                           // normalised input out
    const int cr = lane >> 3, cp = lane & 7;                 // copy pattern: row cr + 4 k, piece cp
    // the conv values of the warp's block are asked for while the last MMAs run
    float4 cin[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int r = cr + 4 * k;
      cin[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row0 + r < M) cin[k] = __ldg(reinterpret_cast<const float4*>(x + (row0 + r) * E + e0 + cp * 4));
    }
    if (ok) ok = mbar_wait(bar_acc, 0, s_abort);             // every MMA has read the ring by now
    tc_fence_after();
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int r = cr + 4 * k;
      *reinterpret_cast<float4*>(blk_a + r * 128 + ((cp ^ (r & 7)) << 4)) = cin[k];
    }
    __syncwarp();
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + cq * 32;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      uint32_t zx[16], za[16];
      tc_ld_32x16(t_row + cc * 16, zx);
      tc_ld_32x16(t_row + kHalf + cc * 16, za);
      tc_wait_ld();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int piece = (cc * 4 + q) ^ (lane & 7);
        const float4 cv = *reinterpret_cast<const float4*>(blk_a + lane * 128 + (piece << 4));
        const float cvv[4] = {cv.x, cv.y, cv.z, cv.w};
        float av[4], xv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = q * 4 + j;
          const int ch = cq * 32 + cc * 16 + n;            // channel within the half
          gate_math<false, true>(cvv[j], __uint_as_float(zx[n]), __uint_as_float(za[n]), s_sp[kHalf + ch],
                           s_sp[2 * kHalf + ch], s_sp[ch], is_reset, av[j], xv[j]);
        }
        *reinterpret_cast<float4*>(blk_a + lane * 128 + (piece << 4)) = make_float4(av[0], av[1], av[2], av[3]);
        *reinterpret_cast<float4*>(blk_x + lane * 128 + (piece << 4)) = make_float4(xv[0], xv[1], xv[2], xv[3]);
      }
    }
    __syncwarp();
    if (ok) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int r = cr + 4 * k;
        if (row0 + r < M) {
          const int off = r * 128 + ((cp ^ (r & 7)) << 4);
          *reinterpret_cast<float4*>(a_out + (row0 + r) * E + e0 + cp * 4) =
              *reinterpret_cast<const float4*>(blk_a + off);
          *reinterpret_cast<float4*>(xn_out + (row0 + r) * E + e0 + cp * 4) =
              *reinterpret_cast<const float4*>(blk_x + off);
        }
      }
    }
  }

  // ------------------------------ teardown --------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *s_abort) atomicExch(&hdr->status, kStatusTimeout);
  if (warp == kEpi + 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(256)
                 : "memory");
  }
}

// Splits the two gate weights [H, 256 (k), 256 (n)] float32 into K-major groups
// [H, 2, 256 (n'), 256 (k)] (rows 0-127 of a group: the x-gate columns of its 128 channels, rows
// 128-255 the a-gate ones), once with the low 13 mantissa bits cleared and once as what they held.
__global__ void pack_gate_weights_tf32_kernel(const float* __restrict__ wx, const float* __restrict__ wa,
                                              int H, float* __restrict__ hi, float* __restrict__ lo) {
  __shared__ float tile[32][33];
  const int group = blockIdx.z, head = group >> 1, half = group & 1;
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;          // n' in [0, 256)
  const float* src = (n0 < kHalf ? wx : wa) + (int64_t)head * kHW * kHW;
  const int chan = half * kHalf + (n0 % kHalf);
  for (int r = threadIdx.y; r < 32; r += 8)                        // r walks k, x walks n
    tile[r][threadIdx.x] = src[(int64_t)(k0 + r) * kHW + chan + threadIdx.x];
  __syncthreads();
  const int64_t base = (int64_t)group * kTN * kHW;
  for (int r = threadIdx.y; r < 32; r += 8) {                      // r walks n', x walks k
    const float v = tile[threadIdx.x][r];
    const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
    hi[base + (int64_t)(n0 + r) * kHW + k0 + threadIdx.x] = h;
    lo[base + (int64_t)(n0 + r) * kHW + k0 + threadIdx.x] = v - h;
  }
}

}  // namespace

size_t gates_tf32_packed_bytes(int H) { return (size_t)H * 2 * kTN * kHW * 4 * 2; }

bool gates_tf32_supported(int dtype, int bw, int64_t M) {
  return dtype == 0 && bw == kHW && M >= 1 && M < ((int64_t)1 << 31);
}

cudaError_t launch_pack_gate_weights_tf32(const void* wx, const void* wa, int H, void* packed_w,
                                          cudaStream_t s) {
  float* hi = static_cast<float*>(packed_w);
  float* lo = hi + (size_t)H * 2 * kTN * kHW;
  pack_gate_weights_tf32_kernel<<<dim3(kHW / 32, kTN / 32, 2 * H), dim3(32, 8), 0, s>>>(
      (const float*)wx, (const float*)wa, H, hi, lo);
  return cudaGetLastError();
}

cudaError_t launch_gates_tf32(const void* c, const void* pos, int pos64, const void* a_param,
                              const void* wx, const void* bx, const void* wa, const void* ba,
                              int64_t M, int H, void* packed_w, bool packed_valid, void* a_out,
                              void* xn_out, void* ws_header, cudaStream_t s) {
  if (M == 0) return cudaSuccess;
  const int E = H * kHW;
  float* hi = static_cast<float*>(packed_w);
  float* lo = hi + (size_t)H * 2 * kTN * kHW;
  if (!packed_valid) {
    cudaError_t err = launch_pack_gate_weights_tf32(wx, wa, H, packed_w, s);
    if (err != cudaSuccess) return err;
  }

  CUtensorMap map_x, map_wh, map_wl;
  if (!tensor_map_2d(&map_x, c, (uint64_t)M, (uint64_t)E, kTM, kKS, kSw128, 4, !kSw128) ||
      !tensor_map_2d(&map_wh, hi, (uint64_t)H * 2 * kTN, kHW, kTN, kKS, kSw128, 4, !kSw128) ||
      !tensor_map_2d(&map_wl, lo, (uint64_t)H * 2 * kTN, kHW, kTN, kKS, kSw128, 4, !kSw128))
    return cudaErrorInvalidValue;
  static PerDeviceOnce once;
  cudaError_t e0 = once.run([] {
    return cudaFuncSetAttribute(gates_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemF);
  });
  if (e0 != cudaSuccess) return e0;
  const dim3 grid((unsigned)((M + kTM - 1) / kTM), (unsigned)(2 * H));
  gates_tf32_kernel<<<grid, kThreadsF, kSmemF, s>>>(
      map_x, map_wh, map_wl, (const float*)c, pos, pos64, (const float*)a_param, (const float*)bx,
      (const float*)ba, M, E, (float*)a_out, (float*)xn_out, reinterpret_cast<WsHeader*>(ws_header));
  return cudaGetLastError();
}

}  // namespace rgk
