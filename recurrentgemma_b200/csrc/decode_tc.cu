// One decode step of the RG-LRU + Conv1D sub-path as a single kernel (bfloat16, heads of width
// 256): recurrentgemma torch/layers.py:469-550 (Conv1D with a cache), 338-353 (gates), 170-177
// (rnn_scan with one token) and the join of torch/modules.py:627-628, 646.
//
// The "tokens" of the contraction are the batch rows.  A CTA serves 128 rows x one quarter of a
// head (64 channels); the four CTAs of a head form a cluster.  The A operand - the conv output of
// the 128 rows for all 256 channels of the head, computed from the new token and the three cached
// rows with the reference's bfloat16 roundings, in the 128-byte-swizzled K-major layout tcgen05
// reads - is built once per cluster: each CTA computes the slice of its own 64 channels and stores it
// into the shared memory of all four (distributed shared memory), while TMA brings the CTA's 64
// x-gate and 64 a-gate weight rows (64 KiB, pre-packed K-major).  Sixteen tcgen05.mma (M 128, N 128, K 16) leave both gates of every channel in TMEM;
// the epilogue does the gate arithmetic, the state update h = a h + x in float32 (stored
// unrounded), the join with gelu(y branch), and writes out / state / shifted conv cache.
//
// Both mbarrier waits are bounded; on expiry WsHeader::status is raised and the CTA leaves.
#include <cuda.h>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tc_common.cuh"

namespace rgk {
namespace {

constexpr int kHeadW = 256;
constexpr int kRowsM = 128;
constexpr int kChanCta = 64;                     // channels per CTA
constexpr int kN = 2 * kChanCta;                 // accumulator columns: 64 x-gate + 64 a-gate
constexpr int kSlices = 4;                       // K slices of 64 channels
constexpr int kASlice = kRowsM * 128;            // 16 KiB
constexpr int kBSlice = kN * 128;                // 16 KiB
constexpr int kOffB = 0;
constexpr int kOffA = kSlices * kBSlice;                       // 65536
constexpr int kOffConst = kOffA + kSlices * kASlice;           // 131072
constexpr int kOffBar = kOffConst + 3 * (kChanCta / 2) * 4;    // two mbarriers
constexpr int kOffTmem = kOffBar + 16;
constexpr int kOffAbort = kOffTmem + 4;
constexpr int kOffLutDec = (kOffAbort + 4 + 15) & ~15;        // {a, multiplier} by log_a (tc_common.cuh)
constexpr int kSmem = kOffLutDec + kLutEntries * 4 + 1024;
constexpr int kThreadsDec = 512;
constexpr int kEpiCols = kChanCta / (kThreadsDec / 128);   // channels per epilogue thread: 16
constexpr uint32_t kIdescDec = tc_idesc_bf16(kRowsM, kN);

__device__ __forceinline__ uint4 mul4(const uint4& a, const uint4& b) {
  return make_uint4(bmul2(a.x, b.x), bmul2(a.y, b.y), bmul2(a.z, b.z), bmul2(a.w, b.w));
}
__device__ __forceinline__ uint4 add4(const uint4& a, const uint4& b) {
  return make_uint4(badd2(a.x, b.x), badd2(a.y, b.y), badd2(a.z, b.z), badd2(a.w, b.w));
}

// kMath: how the gates and the gelu are evaluated (see rgk_internal.h); the fast variant takes
// a = exp(log_a) and the input multiplier from a shared-memory table, built in the prologue.
template <bool kMul, int kMath>
__global__ void __launch_bounds__(kThreadsDec, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __nv_bfloat16* __restrict__ xb,
                 const __nv_bfloat16* __restrict__ yb, const void* __restrict__ pos, int pos64,
                 const __nv_bfloat16* __restrict__ conv_w, const __nv_bfloat16* __restrict__ conv_b,
                 const __nv_bfloat16* __restrict__ a_param, const __nv_bfloat16* __restrict__ bias_x,
                 const __nv_bfloat16* __restrict__ bias_a, const float* h_in,
                 const __nv_bfloat16* cache_in, const void* __restrict__ packed_w, int M, int E,
                 __nv_bfloat16* __restrict__ out, float* h_out,
                 __nv_bfloat16* cache_out, WsHeader* hdr) {
  extern __shared__ uint8_t smem_raw[];
  // aligned by an offset into the shared array, so that the address space stays known to the
  // compiler (shared-memory load/store instructions instead of generic ones)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t s_base = smem_u32(smem);
  uint32_t* s_const = reinterpret_cast<uint32_t*>(smem + kOffConst);
  const uint32_t bar_b = s_base + kOffBar, bar_mma = s_base + kOffBar + 8;
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + kOffTmem);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffAbort);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.x >> 2, quarter = blockIdx.x & 3;
  const int tile = blockIdx.y;
  const int chan0 = head * kHeadW + quarter * kChanCta;   // first channel this CTA produces

  uint32_t* s_lut = reinterpret_cast<uint32_t*>(smem + kOffLutDec);
  if constexpr (kMath == kMathFast)
    for (int i = tid; i < kLutEntries; i += kThreadsDec) s_lut[i] = a_mult_entry(i);
  if (tid == 0) {
    *s_abort = 0;
    mbar_init(bar_b, 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(s_base + kOffTmem), "r"(kN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid < 3 * (kChanCta / 2)) {
    const int which = tid / (kChanCta / 2), pair = tid % (kChanCta / 2);
    const int e = chan0 + 2 * pair;
    uint32_t v;
    if (which == 0) v = *reinterpret_cast<const uint32_t*>(bias_x + e);
    else if (which == 1) v = *reinterpret_cast<const uint32_t*>(bias_a + e);
    else {
      const float s0 = round_bf16(softplus_(__bfloat162float(a_param[e])));
      const float s1 = round_bf16(softplus_(__bfloat162float(a_param[e + 1])));
      // (clamped to the range of the table: beyond it a = exp(log_a) is 0 in float32 either way)
      v = kMath == kMathFast ? pack_bf16x2(fmaxf(-8.0f * s0, kLogAFloor), fmaxf(-8.0f * s1, kLogAFloor))
                             : pack_bf16x2(-8.0f * s0, -8.0f * s1);
    }
    s_const[which * (kChanCta / 2) + pair] = v;
  }
  // What this step reads besides the predecessor's activations - the packed gate weights, the conv
  // window and the state - comes from HBM (26 layers of them do not stay in L2 from one token to
  // the next).  Asking for it to be brought into L2 is harmless whoever wrote it last (L2 is the
  // point of coherence), so it is done before the dependency wait: the CTAs of a row tile split
  // the tile's contiguous cache and state rows, all CTAs the weights.
  if (tid == 32) {
    const int64_t row0 = (int64_t)tile * kRowsM;
    const int64_t rows = min((int64_t)kRowsM, (int64_t)M - row0);
    const int n_x = gridDim.x, n_all = gridDim.x * gridDim.y;
    const int me_all = blockIdx.y * gridDim.x + blockIdx.x;
    auto prefetch_share = [](const void* base, int64_t bytes, int part, int parts) {
      int64_t chunk = ((bytes + parts - 1) / parts + 127) & ~(int64_t)127;
      const int64_t lo = (int64_t)part * chunk;
      if (lo >= bytes) return;
      if (lo + chunk > bytes) chunk = (bytes - lo) & ~(int64_t)15;
      if (chunk > 0)
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;"
                     :: "l"(static_cast<const char*>(base) + lo), "r"((uint32_t)chunk) : "memory");
    };
    prefetch_share(cache_in + row0 * 3 * E, rows * 3 * E * 2, blockIdx.x, n_x);
    prefetch_share(h_in + row0 * E, rows * E * 4, blockIdx.x, n_x);
    prefetch_share(packed_w, (int64_t)E * 2 * kHeadW * 2, me_all, n_all);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  // ---- weights: 64 x-gate rows and 64 a-gate rows of this quarter, per K slice -------------------
  // (After the dependency wait: the packed copy may have been written by the kernel just before.)
  if (tid == 0) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    mbar_expect_tx(bar_b, kSlices * kBSlice);
    const int group_row = (head * 2 + (quarter >> 1)) * 256 + (quarter & 1) * kChanCta;
    for (int k = 0; k < kSlices; ++k) {
      tma_load_2d(s_base + kOffB + k * kBSlice, &map_w, k * 64, group_row, bar_b);
      tma_load_2d(s_base + kOffB + k * kBSlice + kChanCta * 128, &map_w, k * 64, group_row + 128,
                  bar_b);
    }
  }

  // ---- A operand: conv output of 128 rows x the head's 256 channels ------------------------------
  // The four CTAs of a head (a cluster) need the same A tile.  Each computes the K slice of its own
  // 64 channels and stores it into the shared memory of all four: a quarter of the loads and of the
  // arithmetic per CTA.
  {
    const int pk = tid & 7;                       // 16-byte pack inside this CTA's slice of channels
    const int e = chan0 + pk * 8;
    uint4 wv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) wv[k] = *reinterpret_cast<const uint4*>(conv_w + (int64_t)k * E + e);
    const uint4 bv = *reinterpret_cast<const uint4*>(conv_b + e);
    uint32_t a_remote[4];                         // this slice inside each CTA of the cluster
#pragma unroll
    for (int d = 0; d < 4; ++d)
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                   : "=r"(a_remote[d]) : "r"(s_base + kOffA + quarter * kASlice), "r"(d));
    // Everything above (barriers, TMEM, the per-channel constants) is independent of the kernel
    // before this one on the stream, which in a decode loop is the previous layer: with
    // programmatic dependent launch it overlaps that kernel's tail.  The activations below are its
    // output, so wait for it here, then let the next layer's prologue start in turn.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // two rows per thread, their 8 loads all issued before the first use
    constexpr int kPer = kRowsM * 8 / kThreadsDec;     // rows per thread: 2
    constexpr int kRowStep = kThreadsDec / 8;
    uint4 xv[kPer][4];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int r = (tid >> 3) + kRowStep * i;
      const int64_t m = min((int64_t)tile * kRowsM + r, (int64_t)M - 1);   // clamped: never out of range
      const __nv_bfloat16* cr = cache_in + m * 3 * E + e;
      xv[i][0] = *reinterpret_cast<const uint4*>(cr);
      xv[i][1] = *reinterpret_cast<const uint4*>(cr + E);
      xv[i][2] = *reinterpret_cast<const uint4*>(cr + 2 * (int64_t)E);
      xv[i][3] = *reinterpret_cast<const uint4*>(xb + m * E + e);
    }
    // every CTA of the cluster is running before its shared memory is written from outside
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int r = (tid >> 3) + kRowStep * i;
      const int64_t m = (int64_t)tile * kRowsM + r;
      // newest tap first (torch/layers.py:491-517 with prompt_len = 3), then the bias
      uint4 acc = mul4(xv[i][3], wv[3]);
      acc = add4(acc, mul4(xv[i][2], wv[2]));
      acc = add4(acc, mul4(xv[i][1], wv[1]));
      acc = add4(acc, mul4(xv[i][0], wv[0]));
      acc = add4(acc, bv);
      if (m < M) {
        if (cache_out != nullptr) {               // these are this CTA's own channels: shift the cache
          __nv_bfloat16* co = cache_out + m * 3 * E + e;
          *reinterpret_cast<uint4*>(co) = xv[i][1];
          *reinterpret_cast<uint4*>(co + E) = xv[i][2];
          *reinterpret_cast<uint4*>(co + 2 * (int64_t)E) = xv[i][3];
        }
      } else {
        acc = make_uint4(0u, 0u, 0u, 0u);
      }
      const uint32_t off = r * 128 + ((pk ^ (r & 7)) << 4);
#pragma unroll
      for (int d = 0; d < 4; ++d)
        asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};"
                     :: "r"(a_remote[d] + off), "r"(acc.x), "r"(acc.y), "r"(acc.z), "r"(acc.w) : "memory");
    }
  }
  // The tile is complete when all four CTAs have stored their slices: the generic-proxy writes are
  // fenced towards the tensor core's (async) proxy, then released and acquired across the cluster.
  asm volatile("fence.proxy.async;" ::: "memory");
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");

  // ---- MMA ------------------------------------------------------------------------------------------
  if (tid == 0) {
    if (mbar_wait(bar_b, 0, s_abort)) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < kSlices; ++k) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t da = smem_desc_sw128(s_base + kOffA + k * kASlice + ks * 32);
          const uint64_t db = smem_desc_sw128(s_base + kOffB + k * kBSlice + ks * 32);
          tc_mma_bf16(tmem_base, da, db, kIdescDec, (k | ks) != 0 ? 1u : 0u);
        }
      }
      tc_commit(bar_mma);
    }
  }

  // ---- epilogue: 16 warps = 4 TMEM lane quarters x 4 groups of 16 channels ------------------------
  {
    const int lane_base = (warp & 3) * 32, col_grp = warp >> 2;
    const int r = lane_base + lane;
    const int64_t m = (int64_t)tile * kRowsM + r;
    const bool row_ok = m < M;
    const int64_t m_ld = row_ok ? m : 0;
    const bool is_reset = row_ok && pos_is_zero(pos, pos64, m);
    const int e = chan0 + col_grp * kEpiCols;
    // inputs of the state update and of the join, in flight while the MMA runs
    float4 hv[kEpiCols / 4];
    uint4 yv[kEpiCols / 8];
#pragma unroll
    for (int j = 0; j < kEpiCols / 4; ++j)
      hv[j] = *reinterpret_cast<const float4*>(h_in + m_ld * E + e + 4 * j);
    if constexpr (kMul) {
#pragma unroll
      for (int j = 0; j < kEpiCols / 8; ++j)
        yv[j] = *reinterpret_cast<const uint4*>(yb + m_ld * E + e + 8 * j);
    }
    if (mbar_wait(bar_mma, 0, s_abort)) {
      tc_fence_after();
      uint32_t zx[kEpiCols], za[kEpiCols];
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + col_grp * kEpiCols;
      tc_ld_32x16(t_row, zx);
      tc_ld_32x16(t_row + kChanCta, za);
      // conv outputs of these 16 channels: slice `quarter` of the A tile, units col_grp*2, +1
      uint4 cv[kEpiCols / 8];
      const uint8_t* a_row = smem + kOffA + quarter * kASlice + r * 128;
#pragma unroll
      for (int j = 0; j < kEpiCols / 8; ++j)
        cv[j] = *reinterpret_cast<const uint4*>(a_row + (((col_grp * (kEpiCols / 8) + j) ^ (r & 7)) << 4));
      tc_wait_ld();
#pragma unroll
      for (int j = 0; j < kEpiCols / 8; ++j) {
        const uint32_t cp[4] = {cv[j].x, cv[j].y, cv[j].z, cv[j].w};
        const uint32_t yp[4] = {yv[j].x, yv[j].y, yv[j].z, yv[j].w};
        float hn[8];
        uint32_t op[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const int n = j * 8 + p * 2;
          const int pair = (col_grp * kEpiCols + n) >> 1;
          uint32_t a2, xn2;
          if constexpr (kMath == kMathFast) {
            uint32_t gx2, mult2;
            const uint32_t bx2 = s_const[pair];
            gate_tokens<kMathFast, true>(__uint_as_float(zx[n]), __uint_as_float(zx[n + 1]),
                                         __uint_as_float(za[n]), __uint_as_float(za[n + 1]), bx2,
                                         s_const[kChanCta / 2 + pair], bmul2(bx2, 0x3f003f00u),
                                         s_const[kChanCta + pair], a2, gx2, mult2, s_lut);
            if (is_reset) {
              mult2 = 0x3f803f80u;
              a2 = 0u;
            }
            xn2 = bmul2(bmul2(cp[p], gx2), mult2);
          } else {
            gate_pair(__uint_as_float(zx[n]), __uint_as_float(zx[n + 1]), __uint_as_float(za[n]),
                      __uint_as_float(za[n + 1]), s_const[pair], s_const[kChanCta / 2 + pair],
                      s_const[kChanCta + pair], cp[p], is_reset, a2, xn2);
          }
          const float h0v = (p & 1) ? hv[2 * j + (p >> 1)].z : hv[2 * j + (p >> 1)].x;
          const float h1v = (p & 1) ? hv[2 * j + (p >> 1)].w : hv[2 * j + (p >> 1)].y;
          // h = a h + x in float32; the state keeps the unrounded value (torch/layers.py:176-177)
          hn[2 * p] = fmaf(bf16_lo(a2), h0v, bf16_lo(xn2));
          hn[2 * p + 1] = fmaf(bf16_hi(a2), h1v, bf16_hi(xn2));
          op[p] = pack_bf16x2(hn[2 * p], hn[2 * p + 1]);
          if constexpr (kMul) {
            if constexpr (kMath == kMathFast) {
              op[p] = join_gelu2<kMathFast>(op[p], yp[p]);
            } else {
              const float g0 = gelu_tanh_<true>(bf16_lo(yp[p])), g1 = gelu_tanh_<true>(bf16_hi(yp[p]));
              op[p] = bmul2(op[p], pack_bf16x2(g0, g1));
            }
          }
        }
        if (row_ok) {
          *reinterpret_cast<float4*>(h_out + m * E + e + 8 * j) = make_float4(hn[0], hn[1], hn[2], hn[3]);
          *reinterpret_cast<float4*>(h_out + m * E + e + 8 * j + 4) = make_float4(hn[4], hn[5], hn[6], hn[7]);
          *reinterpret_cast<uint4*>(out + m * E + e + 8 * j) = make_uint4(op[0], op[1], op[2], op[3]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *s_abort) atomicExch(&hdr->status, kStatusTimeout);
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(kN)
                 : "memory");
  }
}



}  // namespace

cudaError_t launch_path_decode_tc(const void* xb, const void* yb, const void* pos, int pos64,
                                  const void* conv_w, const void* conv_b, const void* a_param,
                                  const void* bx, const void* ba, const void* packed_w,
                                  const float* h_in, const void* cache_in, int64_t B, int H,
                                  void* out, float* h_out, void* cache_out, void* ws_header,
                                  cudaStream_t s, int math) {
  if (B == 0) return cudaSuccess;
  using T_ = __nv_bfloat16;
  CUtensorMap map_w;
  if (!tensor_map_2d(&map_w, packed_w, (uint64_t)H * 2 * 256, 256, kChanCta, 64, true))
    return cudaErrorInvalidValue;
  static PerDeviceOnce once;
  cudaError_t e0 = once.run([] {
    cudaError_t e;
#define RGK_DEC_ATTR(MUL, MATH)                                                                 \
    if ((e = cudaFuncSetAttribute(decode_tc_kernel<MUL, MATH>,                                  \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem)) != cudaSuccess) return e
    RGK_DEC_ATTR(true, kMathExact);
    RGK_DEC_ATTR(true, kMathFast);
    RGK_DEC_ATTR(false, kMathExact);
    RGK_DEC_ATTR(false, kMathFast);
#undef RGK_DEC_ATTR
    return cudaSuccess;
  });
  if (e0 != cudaSuccess) return e0;
  const dim3 grid((unsigned)(H * 4), (unsigned)((B + kRowsM - 1) / kRowsM));
  const int E = H * kHeadW;
  // Launched with programmatic stream serialization: the kernel may start while its predecessor
  // on the stream is still draining; it orders itself with griddepcontrol.wait.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreadsDec);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;      // the four channel quarters of a head
  attr[1].val.clusterDim.x = 4;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
#define RGK_DEC(MUL, MATH)                                                                         \
  cudaLaunchKernelEx(&cfg, decode_tc_kernel<MUL, MATH>, map_w, (const T_*)xb, (const T_*)yb, pos,  \
                     pos64, (const T_*)conv_w, (const T_*)conv_b, (const T_*)a_param, (const T_*)bx, \
                     (const T_*)ba, h_in, (const T_*)cache_in, packed_w, (int)B, E, (T_*)out,      \
                     h_out, (T_*)cache_out, reinterpret_cast<WsHeader*>(ws_header))
  cudaError_t lerr;
  if (math == kMathExact) lerr = yb ? RGK_DEC(true, kMathExact) : RGK_DEC(false, kMathExact);
  else lerr = yb ? RGK_DEC(true, kMathFast) : RGK_DEC(false, kMathFast);
  if (lerr != cudaSuccess) return lerr;
#undef RGK_DEC
  return cudaGetLastError();
}

}  // namespace rgk
