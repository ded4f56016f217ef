// RG-LRU forward in ONE kernel with channel-major accumulators: the block-diagonal gate projections
// run on tcgen05 as  D[channel, token] = W[channel, k] . C[token, k]^T,  so that a TMEM lane is a
// channel and its columns are consecutive tokens.  An epilogue thread then owns one channel and a
// run of 32 tokens: gate arithmetic, the linear recurrence and the join with the other branch all
// happen in its registers, in time order, with no transposition (recurrentgemma torch/layers.py:
// 127-137, 313-365, 140-191; join of torch/modules.py:627-628, 646).  The recurrence coefficients a
// and the normalised input never reach HBM.  bfloat16, heads of width 256, any sequence length
// (the last time tile of a sequence may be partial: the copy engine fills rows past the end with
// zeros and drops them from the stores, and those tokens act as the identity map).
//
// Units of work: 128 consecutive tokens of one sequence x one half of a head (128 channels).  Units
// are numbered time-major and dealt out round-robin to persistent CTAs, one per SM, so the unit that
// produces a carry has normally finished one round before the unit that consumes it starts.
//
// Roles in a CTA (18 warps):
//   producer  one thread: per K-slice of 64 the conv-output tile (128 tokens x 64, operand B) and the
//             packed gate weights (256 gate rows x 64, operand A) by TMA into a 3-stage ring;
//   MMA       one thread: per K-step two tcgen05.mma M128 N128 (x-gate rows, a-gate rows) into one
//             of two TMEM accumulator sets (2 x 128 columns each);
//   epilogue  16 warps = 4 channel quarters (the warp's TMEM lane quarter) x 4 token quarters.
//             A warp fetches its own 32 x 32 tiles of the conv output and of the other branch by
//             TMA (64-byte swizzle) into 2 KiB buffers, transposes each in place (ldmatrix.trans +
//             stmatrix) so that a thread finds the 32 tokens of its channel as four 16-byte pieces,
//             writes its outputs the same way, transposes back and hands the tile to a TMA store:
//             every global access of the kernel is a bulk tensor copy, every shared-memory access
//             of the tiles a 16-byte one.
// Per unit an epilogue thread: tcgen05.ld of 2 x 16 columns -> gate arithmetic on token pairs in
// packed bfloat16 with the reference's roundings -> (a, x) kept packed in 32 registers while the
// 32-token map (P, H): h -> P h + H is accumulated -> the four token quarters of a channel quarter
// meet at a 128-thread named barrier; the last one publishes the tile's map, resolves the incoming
// state (decoupled look-back over earlier time tiles, normally one already inclusive record) and
// publishes the inclusive state -> second named barrier -> replay from registers with the true
// incoming state, join, 16-byte stores into the output tile.
// All waits (mbarriers, look-back flags) are bounded; on expiry WsHeader::status is raised, the
// affected values are taken as zero and the kernel runs to completion.
#include <cuda.h>

#include "rgk_common.cuh"
#include "rgk_internal.h"
#include "tc_common.cuh"

namespace rgk {
namespace {

constexpr int kHW = 256;                 // head width = K
constexpr int kUT = 128;                 // tokens per unit (MMA N)
constexpr int kUC = 128;                 // channels per unit (MMA M)
constexpr int kKB = 64;                  // K per ring stage
constexpr int kKBlocks = kHW / kKB;      // 4
constexpr int kRing = 3;
constexpr int kCBytes = kUT * kKB * 2;         // 16 KiB: conv-output slice (operand B)
constexpr int kWBytes = 2 * kUC * kKB * 2;     // 32 KiB: x-gate rows then a-gate rows (operand A)
constexpr int kStage = kCBytes + kWBytes;
constexpr int kEpi = 16;
constexpr int kThreads = (kEpi + 2) * 32;
// With the Conv1D fused (kConv): two more warps turn the block input into the conv-output operand.
// The ring then has two stages; the room of the third holds two staging buffers for the input rows
// of a K-slice (the unit's 128 tokens and the three before them, 64 channels).
constexpr int kConvWarps = 2;
constexpr int kThreadsConv = (kEpi + 2 + kConvWarps) * 32;
constexpr int kRingConv = 2;
constexpr int kXRows = kUT + 3;
constexpr int kXBytes = kXRows * kKB * 2;      // 16768
constexpr int kXStage = 17 * 1024;
constexpr int kOffXs = kRingConv * kStage;
static_assert(kOffXs + 2 * kXStage <= kRing * kStage, "the staging buffers overlap the warp tiles");
constexpr int kSub = 32;                 // a warp's tile: 32 tokens x 32 channels
constexpr int kSubBytes = kSub * kSub * 2;
constexpr int kOffRing = 0;
constexpr int kOffTiles = kRing * kStage;                      // per warp: conv tile, then y/out tile
constexpr int kOffQmap = kOffTiles + kEpi * 2 * kSubBytes;     // float2 [2 parity][4 chq][3 tq][32]
constexpr int kOffHin = kOffQmap + 2 * 4 * 3 * 32 * 8;         // float  [2 parity][4 chq][32]
constexpr int kOffKnown = kOffHin + 2 * 4 * 32 * 4;              // int    [2 parity][4 chq]
constexpr int kOffBar = kOffKnown + 2 * 4 * 4;
constexpr int kNumBar = 2 * kRing + 4 + 2 * kEpi + 5;        // + staging full[2], empty[2], conv tiles free
constexpr int kOffTmem = kOffBar + kNumBar * 8;
constexpr int kOffAbort = kOffTmem + 4;
constexpr int kOffLut = (kOffAbort + 4 + 15) & ~15;            // {a, multiplier} by log_a, see tc_common.cuh
constexpr int kSmem = kOffLut + kLutEntries * 4 + 1024;
static_assert(kSmem <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");
constexpr uint32_t kIdesc = tc_idesc_bf16(kUC, kUT);
constexpr unsigned kLookbackSpins = 1u << 20;

__device__ __forceinline__ uint4 mul4(const uint4& a, const uint4& b) {
  return make_uint4(bmul2(a.x, b.x), bmul2(a.y, b.y), bmul2(a.z, b.z), bmul2(a.w, b.w));
}
__device__ __forceinline__ uint4 add4(const uint4& a, const uint4& b) {
  return make_uint4(badd2(a.x, b.x), badd2(a.y, b.y), badd2(a.z, b.z), badd2(a.w, b.w));
}

// An inclusive state travels as one 64-bit word per channel {h, token}: one store, one load, and a
// reader that finds the token has the value, without a flag or a fence.
constexpr unsigned long long kToken = 1ull << 32;
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}

// The map of one (unit, channel quarter) travels the same way: two words per channel, {P, token}
// and {H, token}.  A reader that looks back over several earlier tiles asks for the state words and
// the map words of all of them at once and uses whatever has arrived: one round trip to memory.
constexpr int kLookback = 2;             // earlier tiles asked for per round trip (more cost registers)

// In-place transposition of a warp's 32 x 32 bfloat16 tile (rows of 64 bytes, 64-byte swizzle:
// 16-byte piece j of row r at position j ^ ((r >> 1) & 3)).  ldmatrix.trans hands thread T of the
// warp, for each 8 x 8 block, the elements (rows 2 (T % 4) and 2 (T % 4) + 1, column T / 4) packed
// into one register - the fragment (row T / 4, columns 2 (T % 4), + 1) of the transposed block,
// which stmatrix stores.  The whole tile sits in registers between the two, so it is written back
// over itself, rows and columns exchanged, in the same swizzled layout.  Every access is
// conflict-free.  ld_base = tile + lane * 64 + (((lane >> 1) & 3) << 4): the address of the lane's
// own row at piece 0; st_base = tile + (lane & 7) * 64 + (((lane >> 3) ^ ((lane >> 1) & 3)) << 4).
__device__ __forceinline__ void transpose_tile(uint32_t ld_base, uint32_t st_base) {
  uint32_t r[4][4];
#pragma unroll
  for (int q = 0; q < 4; ++q)
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[q][0]), "=r"(r[q][1]), "=r"(r[q][2]), "=r"(r[q][3])
                 : "r"(ld_base ^ (uint32_t)(q << 4)) : "memory");
  __syncwarp();
#pragma unroll
  for (int q = 0; q < 4; ++q)
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};"
                 :: "r"(st_base + (uint32_t)(q * 512)), "r"(r[q][0]), "r"(r[q][1]), "r"(r[q][2]),
                    "r"(r[q][3]) : "memory");
  __syncwarp();
}
// Piece k (tokens 8 k .. 8 k + 7 as four token pairs) of the lane's own row of a transposed tile.
__device__ __forceinline__ uint4 lds_piece(uint32_t ld_base, int k) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(ld_base ^ (uint32_t)(k << 4)) : "memory");
  return v;
}
__device__ __forceinline__ void sts_piece(uint32_t ld_base, int k, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
               :: "r"(ld_base ^ (uint32_t)(k << 4)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// 16 tokens of one channel: gates from the accumulators, (a, x) packed per token pair, and the
// running map (P, H) of the thread's tokens.  c holds the conv outputs of the 16 tokens as 8 token
// pairs; `rs` holds the reset bits of the 16 tokens, `inv` the bits of tokens past the end of the
// sequence (the kResets variant handles both; the other one has no branch inside the unrolled loop,
// so that the compiler interleaves the eight independent pairs).
template <bool kResets, int kMath>
__device__ __forceinline__ void gates_16(const uint32_t (&zx)[16], const uint32_t (&za)[16],
                                         const uint32_t (&c)[8], uint32_t bx2, uint32_t ba2, uint32_t hbx2,
                                         uint32_t m8sp2, uint32_t rs, uint32_t inv, uint32_t* a_out,
                                         uint32_t* x_out, float& P, float& H, const uint32_t* lut) {
#pragma unroll
  for (int jp = 0; jp < 8; ++jp) {
    uint32_t a2, gx2, mult2;
    gate_tokens<kMath, true>(__uint_as_float(zx[2 * jp]), __uint_as_float(zx[2 * jp + 1]),
                             __uint_as_float(za[2 * jp]), __uint_as_float(za[2 * jp + 1]), bx2, ba2,
                             hbx2, m8sp2, a2, gx2, mult2, lut);
    if constexpr (kResets) {
      // a token that starts a document: a = 0, multiplier = 1 (torch/layers.py:343-350, 166)
      const uint32_t keep = (((rs >> (2 * jp)) & 1u) ? 0u : 0x0000ffffu) |
                            (((rs >> (2 * jp + 1)) & 1u) ? 0u : 0xffff0000u);
      a2 &= keep;
      mult2 = (mult2 & keep) | (0x3f803f80u & ~keep);
      // a token past the end of the sequence: the identity map (a = 1, x = 0)
      const uint32_t live = (((inv >> (2 * jp)) & 1u) ? 0u : 0x0000ffffu) |
                            (((inv >> (2 * jp + 1)) & 1u) ? 0u : 0xffff0000u);
      a2 = (a2 & live) | (0x3f803f80u & ~live);
      mult2 = (mult2 & live) | (0x3f803f80u & ~live);
      gx2 &= live;
    }
    const uint32_t x2 = bmul2(bmul2(c[jp], gx2), mult2);
    a_out[jp] = a2;
    x_out[jp] = x2;
    const float a0 = bf16_lo(a2), a1 = bf16_hi(a2);
    // the pair as one map, then composed: keeps the dependent chain at one step per pair
    const float p2 = a0 * a1, h2 = fmaf(a1, bf16_lo(x2), bf16_hi(x2));
    H = fmaf(p2, H, h2);
    P *= p2;
  }
}

// Decoupled look-back of one channel (lane): composes the published maps of earlier tiles of the
// chain, nearest first, until a tile with a known state (or the start of the sequence) is met, and
// returns the state entering tile tt.
__device__ __forceinline__ float look_back(const unsigned long long* agg, const unsigned long long* incl,
                                        const float* h0, int64_t rec, int tt, int per_tt, int b, int E,
                                        int chan, int lane, int use_agg, bool* timed_out_p,
                                        int64_t n_words, int64_t n_state, int* status) {
  float hin = 0.0f;
  bool timed_out = false;
  {
    float Pc = 1.0f, Hc = 0.0f;
    int pred = tt - 1;                 // the nearest tile not yet absorbed
    bool done = false;
    unsigned spins = 0;
    const int depth = use_agg ? kLookback : 1;
    while (!done) {
      unsigned long long wi[kLookback], wp[kLookback], wh[kLookback];
#pragma unroll
      for (int i = 0; i < kLookback; ++i) {
        const int pt = pred - i;
        wi[i] = 0ull; wp[i] = 0ull; wh[i] = 0ull;
        if (i < depth && pt >= 0) {
          const int64_t rp = (rec - (int64_t)(tt - pt) * per_tt * 4) * kSub + lane;
          if (RGK_IN_RANGE(rp, n_words, status)) {
            wi[i] = ld_relaxed_u64(incl + rp);
            if (use_agg) {
              wp[i] = ld_relaxed_u64(agg + rp * 2);
              wh[i] = ld_relaxed_u64(agg + rp * 2 + 1);
            }
          }
        }
      }
      bool progress = false;
#pragma unroll
      for (int i = 0; i < kLookback; ++i) {
        if (!done && pred >= 0 && i < depth) {
          // entries of this batch are consumed strictly in order: entry i belongs to `pred` only
          // while every earlier entry was absorbed
          if ((wi[i] >> 32) == 1ull) {
            hin = fmaf(Pc, __uint_as_float((uint32_t)wi[i]), Hc);
            done = true;
            progress = true;
          } else if ((wp[i] >> 32) == 1ull && (wh[i] >> 32) == 1ull) {
            Hc = fmaf(Pc, __uint_as_float((uint32_t)wh[i]), Hc);
            Pc *= __uint_as_float((uint32_t)wp[i]);
            --pred;
            progress = true;
          } else {
            break;
          }
        }
      }
      if (!done && pred < 0) {
        // every tile back to the start of the sequence was absorbed as a map
        const float hs = (h0 != nullptr && RGK_IN_RANGE((int64_t)b * E + chan, n_state, status))
                             ? h0[(int64_t)b * E + chan] : 0.0f;
        hin = fmaf(Pc, hs, Hc);
        done = true;
      }
      if (!done && !progress) {
        if (++spins > kLookbackSpins) { timed_out = true; break; }
        __nanosleep(32);
      }
    }
  }
  *timed_out_p = timed_out;
  return hin;
}

// Position of a unit (time tile, sequence, half head), advanced by the grid size without divisions.
struct UnitPos {
  int tt, b, grp;
};
struct UnitStep {
  int d_tt, d_b, d_g, B, groups;
  __device__ __forceinline__ void advance(UnitPos& u) const {
    u.grp += d_g;
    if (u.grp >= groups) { u.grp -= groups; u.b += 1; }
    u.b += d_b;
    if (u.b >= B) { u.b -= B; u.tt += 1; }
    u.tt += d_tt;
  }
};

// kJoin 0: out = y, 1: out = y * gelu_tanh(yb), 2: out = y * yb;  kMath: see tc_common.cuh
// kConv: map_c is a map of the block input xb (boxes of 131 rows x 64 channels, no swizzle) and the
// kernel computes the Conv1D (conv_w [4, E], conv_b [E]) itself.
template <int kJoin, int kMath, bool kConv>
__global__ void __launch_bounds__(kConv ? kThreadsConv : kThreads, 1)
rglru_chan_kernel(const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_w,
                  const __grid_constant__ CUtensorMap map_ct, const __grid_constant__ CUtensorMap map_yt,
                  const __grid_constant__ CUtensorMap map_ot, const void* __restrict__ pos, int pos64,
                  const __nv_bfloat16* __restrict__ bias_x, const __nv_bfloat16* __restrict__ bias_a,
                  const __nv_bfloat16* __restrict__ m8sp, const float* __restrict__ h0, int B, int T_,
                  int E, int groups, int n_units, float* __restrict__ h_last, WsHeader* hdr,
                  unsigned long long* agg, unsigned long long* incl, int use_agg,
                  const __nv_bfloat16* __restrict__ conv_w, const __nv_bfloat16* __restrict__ conv_b) {
  extern __shared__ uint8_t smem_raw[];
  // aligned by an offset into the shared array, so that the address space stays known to the
  // compiler (shared-memory load/store instructions instead of generic ones)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar0 = s_base + kOffBar;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kRing + s); };
  auto bar_acc_full = [&](int s) { return bar0 + 8u * (2 * kRing + s); };
  auto bar_acc_empty = [&](int s) { return bar0 + 8u * (2 * kRing + 2 + s); };
  auto bar_ct = [&](int w) { return bar0 + 8u * (2 * kRing + 4 + w); };
  auto bar_yt = [&](int w) { return bar0 + 8u * (2 * kRing + 4 + kEpi + w); };
  auto bar_xs_full = [&](int s) { return bar0 + 8u * (2 * kRing + 4 + 2 * kEpi + s); };
  auto bar_xs_empty = [&](int s) { return bar0 + 8u * (2 * kRing + 4 + 2 * kEpi + 2 + s); };
  const uint32_t bar_cfree = bar0 + 8u * (2 * kRing + 4 + 2 * kEpi + 4);
  constexpr int kR = kConv ? kRingConv : kRing;          // ring stages in use
  constexpr int kAllThreads = kConv ? kThreadsConv : kThreads;
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + kOffTmem);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_t = (T_ + kUT - 1) / kUT;
  const int per_tt = B * groups;                         // units per time tile
  const int n_my = (n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  // a = exp(log_a) and the input multiplier by log_a: computed once per CTA with the very
  // operations the gate arithmetic would use, so that looking them up changes no bit
  uint32_t* s_lut = reinterpret_cast<uint32_t*>(smem + kOffLut);
  for (int i = threadIdx.x; i < kLutEntries; i += kAllThreads) s_lut[i] = a_mult_entry(i);
  if (threadIdx.x == 0) {
    *s_abort = 0;
    // with the conv fused a stage is full when the weights have landed AND the conv warps have
    // written their slice
    for (int s = 0; s < kRing; ++s) { mbar_init(bar_full(s), kConv ? 2 : 1); mbar_init(bar_empty(s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(bar_xs_full(s), 1); mbar_init(bar_xs_empty(s), 1); }
    mbar_init(bar_cfree, kEpi);
    for (int s = 0; s < 2; ++s) { mbar_init(bar_acc_full(s), 1); mbar_init(bar_acc_empty(s), kEpi); }
    for (int w = 0; w < kEpi; ++w) { mbar_init(bar_ct(w), 1); mbar_init(bar_yt(w), 1); }
    mbar_fence_init();
  }
  if (warp == kEpi + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(s_base + kOffTmem), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == kEpi) {
    // ------------------------------ TMA producer of the MMA operands ------------------------------
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int t = 0; t < n_my && ok; ++t) {
        const int u = blockIdx.x + t * gridDim.x;
        const int tt = u / per_tt, rem = u - tt * per_tt;
        const int b = rem / groups, grp = rem - b * groups;
        for (int kb = 0; kb < kKBlocks; ++kb, ++it) {
          if constexpr (kConv) {
            // the input rows of this K-slice for the conv warps (rows before the sequence and past
            // its end read as zero: the first coordinate may be negative)
            const int xs = it & 1;
            ok = mbar_wait(bar_xs_empty(xs), ((it >> 1) & 1) ^ 1, s_abort);
            if (!ok) break;
            mbar_expect_tx(bar_xs_full(xs), kXBytes);
            tma_load_3d(s_base + kOffXs + xs * kXStage, &map_c, (grp >> 1) * kHW + kb * kKB, tt * kUT - 3,
                        b, bar_xs_full(xs));
          }
          const int s = it % kR;
          ok = mbar_wait(bar_empty(s), ((it / kR) & 1) ^ 1, s_abort);
          if (!ok) break;
          if constexpr (kConv) {
            mbar_expect_tx(bar_full(s), kWBytes);
          } else {
            mbar_expect_tx(bar_full(s), kStage);
            tma_load_3d(s_base + kOffRing + s * kStage, &map_c, (grp >> 1) * kHW + kb * kKB, tt * kUT, b,
                        bar_full(s));
          }
          tma_load_2d(s_base + kOffRing + s * kStage + kCBytes, &map_w, kb * kKB, grp * 2 * kUC,
                      bar_full(s));
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
        for (int kb = 0; kb < kKBlocks; ++kb, ++it) {
          const int s = it % kR;
          ok = mbar_wait(bar_full(s), (it / kR) & 1, s_abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t c0 = s_base + kOffRing + s * kStage, w0 = c0 + kCBytes;
#pragma unroll
          for (int ks = 0; ks < kKB / 16; ++ks) {
            const uint32_t acc = (kb | ks) != 0 ? 1u : 0u;
            const uint64_t bdesc = smem_desc_sw128(c0 + ks * 32);
            tc_mma_bf16(tmem_base + as * 2 * kUT, smem_desc_sw128(w0 + ks * 32), bdesc, kIdesc, acc);
            tc_mma_bf16(tmem_base + as * 2 * kUT + kUT, smem_desc_sw128(w0 + kUC * 128 + ks * 32), bdesc,
                        kIdesc, acc);
          }
          tc_commit(bar_empty(s));
        }
        if (ok) tc_commit(bar_acc_full(as));
      }
    }
  } else if (kConv && warp >= kEpi + 2) {
    // ------------------------------ Conv1D (torch/layers.py:447-529) ------------------------------
    // Per K-slice (64 channels of the head) the 64 threads own one 16-byte pack of channels (8) x
    // a run of 16 tokens (8 runs): 19 input rows from the staging buffer through a sliding window,
    // four products and four sums per pack in packed bfloat16 (each rounds where torch does), the
    // result into the slice of the MMA operand (128-byte swizzle) and, for the 128 channels of
    // this unit's half head, into the epilogue warps' conv tiles (rows of 64 bytes, 64-byte
    // swizzle), as the copy engine would have delivered them.
    const int ctid = (int)threadIdx.x - (kEpi + 2) * 32;
    const int pk = ctid & 7, tg = ctid >> 3;
    unsigned it = 0;
    bool ok = true;
    for (int t = 0; t < n_my && ok; ++t) {
      const int u = blockIdx.x + t * gridDim.x;
      const int tt = u / per_tt, rem = u - tt * per_tt;
      const int b = rem / groups, grp = rem - b * groups;
      const int head = grp >> 1, half = grp & 1;
      // nz bit j: token tt*128 + tg*16 - 2 + j starts no document (tokens outside the sequence
      // count as set: their rows are zero, so their taps add nothing).  A warp covers 64 tokens
      // and the two before them: three coalesced loads and ballots, then every thread cuts out
      // the 18 bits of its run.
      unsigned nz;
      {
        const int wl = ctid >> 5, cl = ctid & 31;
        const int base = tt * kUT + wl * 64 - 2;
        unsigned word[3];
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          const int tok = base + q * 32 + cl;
          const bool inside = tok >= 0 && tok < T_ && (q < 2 || cl < 2);
          const bool starts = inside && pos_is_zero(pos, pos64, (int64_t)b * T_ + (inside ? tok : 0));
          word[q] = __ballot_sync(0xffffffffu, !starts);
        }
        const int off = (cl >> 3) * 16;               // first bit of this thread's run
        const unsigned long long lo = (unsigned long long)word[0] | ((unsigned long long)word[1] << 32);
        unsigned long long v = lo >> off;
        if (off == 48) v |= (unsigned long long)(word[2] & 3u) << 16;
        nz = (unsigned)v & 0x3ffffu;
      }
      const bool plain = nz == 0x3ffffu;
      for (int kb = 0; kb < kKBlocks && ok; ++kb, ++it) {
        const int xs = it & 1, s = it % kR;
        const bool mine = (kb >> 1) == half;         // a slice of this unit's own 128 channels
        const int e = head * kHW + kb * kKB + pk * 8;
        uint4 wv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) wv[k] = __ldg(reinterpret_cast<const uint4*>(conv_w + (int64_t)k * E + e));
        const uint4 bv = __ldg(reinterpret_cast<const uint4*>(conv_b + e));
        ok = mbar_wait(bar_xs_full(xs), (it >> 1) & 1, s_abort);
        if (ok) ok = mbar_wait(bar_empty(s), ((it / kR) & 1) ^ 1, s_abort);
        // the epilogue warps have taken the previous unit's conv tiles out of their buffers
        if (ok && mine && t > 0 && (kb & 1) == 0) ok = mbar_wait(bar_cfree, (t - 1) & 1, s_abort);
        if (!ok) break;
        // the staging rows are read with loads the compiler may move across the stores below (the
        // buffers are disjoint), so that the rows of a run are in flight together
        uint32_t xrow = s_base + kOffXs + xs * kXStage + (tg * 16) * (kKB * 2) + pk * 16;
        asm volatile("" : "+r"(xrow) :: "memory");   // the loads below stay behind the waits above
        auto lds16 = [](uint32_t addr) {
          uint4 v;
          asm("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
          return v;
        };
        uint8_t* c_op = smem + kOffRing + s * kStage;
        uint4 x0 = lds16(xrow);
        uint4 x1 = lds16(xrow + kKB * 2);
        uint4 x2 = lds16(xrow + 2 * kKB * 2);
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          const uint4 x3 = lds16(xrow + (r + 3) * (kKB * 2));
          // newest tap first; tap s survives while rows t-s+1 .. t start no document
          uint4 acc = mul4(x3, wv[3]);
          if (plain) {
            acc = add4(acc, mul4(x2, wv[2]));
            acc = add4(acc, mul4(x1, wv[1]));
            acc = add4(acc, mul4(x0, wv[0]));
          } else {
            const bool n0 = (nz >> (r + 2)) & 1u, n1 = (nz >> (r + 1)) & 1u, n2 = (nz >> r) & 1u;
            if (n0) acc = add4(acc, mul4(x2, wv[2]));
            if (n0 && n1) acc = add4(acc, mul4(x1, wv[1]));
            if (n0 && n1 && n2) acc = add4(acc, mul4(x0, wv[0]));
          }
          acc = add4(acc, bv);
          const int row = tg * 16 + r;               // token of the unit
          *reinterpret_cast<uint4*>(c_op + row * 128 + ((pk ^ (row & 7)) << 4)) = acc;
          if (mine) {
            const int w_dst = (row >> 5) * 4 + (kb & 1) * 2 + (pk >> 2);   // token quarter, channel quarter
            const int rr = row & 31, piece = pk & 3;
            *reinterpret_cast<uint4*>(smem + kOffTiles + w_dst * 2 * kSubBytes + rr * 64 +
                                      ((piece ^ ((rr >> 1) & 3)) << 4)) = acc;
          }
          x0 = x1; x1 = x2; x2 = x3;
        }
        // the operand slice is read by the tensor core (async proxy), the staging buffer is
        // overwritten by the copy engine: both after this thread's generic accesses
        fence_proxy_async();
        named_bar_sync(5, kConvWarps * 32);
        if (ctid == 0) {
          mbar_arrive(bar_full(s));
          mbar_arrive(bar_xs_empty(xs));
          if (mine && (kb & 1) == 1)
            for (int w = 0; w < kEpi; ++w) mbar_arrive(bar_ct(w));
        }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------------------------------
    const int chq = warp & 3;                // channel quarter = TMEM lane quarter of this warp
    const int tq = warp >> 2;                // token quarter: tokens 32 tq .. 32 tq + 31 of the unit
    const int set_id = 1 + chq;              // named barrier of the four token quarters
    const uint32_t tile_c_s = s_base + kOffTiles + warp * 2 * kSubBytes, tile_y_s = tile_c_s + kSubBytes;
    // addresses of the in-place transposition and of the lane's own row (see transpose_tile)
    const uint32_t row_off = lane * 64 + (((lane >> 1) & 3) << 4);
    const uint32_t st_off = (lane & 7) * 64 + (((lane >> 3) ^ ((lane >> 1) & 3)) << 4);
    bool ok = true;                          // false once a bounded wait expired: later waits are skipped
    // extents of the record arrays and of the state tensors, for the range checks of the checks build
    const int64_t n_words = (int64_t)n_units * 4 * kSub, n_state = (int64_t)B * E;
    (void)n_words; (void)n_state;

    // unit positions without divisions in the loop
    UnitStep step;
    step.B = B; step.groups = groups;
    step.d_tt = (int)gridDim.x / per_tt;
    {
      const int d_rem = (int)gridDim.x - step.d_tt * per_tt;
      step.d_b = d_rem / groups;
      step.d_g = d_rem - step.d_b * groups;
    }
    UnitPos cur, nxt;
    {
      const int u = blockIdx.x;
      cur.tt = u / per_tt;
      const int rem = u - cur.tt * per_tt;
      cur.b = rem / groups;
      cur.grp = rem - cur.b * groups;
    }
    auto chan0 = [&](const UnitPos& u) { return (u.grp >> 1) * kHW + (u.grp & 1) * kUC + chq * kSub; };
    // whether this lane's token of a unit starts a document (tokens past the end do not)
    auto lane_reset = [&](const UnitPos& u) {
      const int tok = u.tt * kUT + tq * kSub + lane;
      return tok < T_ && pos_is_zero(pos, pos64, (int64_t)u.b * T_ + tok);
    };
    if (!kConv && lane == 0 && n_my > 0) {
      mbar_expect_tx(bar_ct(warp), kSubBytes);
      tma_load_3d(tile_c_s, &map_ct, chan0(cur), cur.tt * kUT + tq * kSub, cur.b, bar_ct(warp));
    }
    // whether this lane's token of the next unit starts a document, and the constants of this
    // lane's channel in the next unit (gate biases, -8 softplus(a_param)): asked for a unit ahead
    bool reset_next = n_my > 0 ? lane_reset(cur) : false;
    uint32_t bxv = 0u, bav = 0u, spv = 0u;
    auto load_consts = [&](const UnitPos& u) {
      const int e = chan0(u) + lane;
      bxv = __ldg(reinterpret_cast<const uint16_t*>(bias_x) + e);
      bav = __ldg(reinterpret_cast<const uint16_t*>(bias_a) + e);
      spv = __ldg(reinterpret_cast<const uint16_t*>(m8sp) + e);
    };
    if (n_my > 0) load_consts(cur);

    for (int t = 0; t < n_my; ++t) {
      const int as = t & 1, par = t & 1;
      const int tt = cur.tt, b = cur.b;
      const int e0 = chan0(cur);                                          // first channel of the warp
      const int tok0 = tt * kUT + tq * kSub;                              // first token of the warp
      const int64_t rec = ((int64_t)(tt * per_tt + b * groups + cur.grp)) * 4 + chq;
      nxt = cur;
      step.advance(nxt);
      float2* s_qmap = reinterpret_cast<float2*>(smem + kOffQmap) + ((par * 4 + chq) * 3) * 32;
      float* s_hin = reinterpret_cast<float*>(smem + kOffHin) + (par * 4 + chq) * 32;
      volatile int* s_known = reinterpret_cast<volatile int*>(smem + kOffKnown) + (par * 4 + chq);

      const uint32_t resets = __ballot_sync(0xffffffffu, reset_next);
      // tokens of this warp past the end of the sequence (only in a sequence's last time tile)
      const int n_live = T_ - tok0;
      const uint32_t invalid = n_live >= 32 ? 0u : (n_live <= 0 ? 0xffffffffu : (0xffffffffu << n_live));
      const uint32_t bx2 = bxv | (bxv << 16), ba2 = bav | (bav << 16), m8sp2 = spv | (spv << 16);
      const uint32_t hbx2 = bmul2(bx2, 0x3f003f00u);

      // the last token quarter asks for its predecessor's inclusive state now (normally published
      // most of a round ago) and looks at the answer after the gate arithmetic
      float hin_pref = 0.0f;
      bool have_hin = tt == 0;
      unsigned long long pre = 0ull;
      if (tq == 3) {
        if (tt == 0) {
          if (h0 != nullptr && RGK_IN_RANGE((int64_t)b * E + e0 + lane, n_state, &hdr->status))
            hin_pref = h0[(int64_t)b * E + e0 + lane];
        } else if (RGK_IN_RANGE((rec - (int64_t)per_tt * 4) * kSub + lane, n_words, &hdr->status)) {
          pre = ld_relaxed_u64(incl + (rec - (int64_t)per_tt * 4) * kSub + lane);
        }
      }

      // ---- gates of the thread's 32 tokens, 16 at a time ------------------------------------------
      if (ok) ok = mbar_wait(bar_acc_full(as), (t >> 1) & 1, s_abort);
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(chq * 32) << 16) + as * 2 * kUT + tq * kSub;
      uint32_t zx[16], za[16];
      tc_ld_32x16(t_row, zx);
      tc_ld_32x16(t_row + kUT, za);
      // while the accumulator columns are on their way from tensor memory: the conv tile is
      // transposed in place, a thread then finds its channel's 32 tokens in its own row
      if (ok) ok = mbar_wait(bar_ct(warp), t & 1, s_abort);
      transpose_tile(tile_c_s + row_off, tile_c_s + st_off);
      uint32_t a_pk[16], x_pk[16];
      float P = 1.0f, H = 0.0f;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t c[8];
        if (half == 1) {
          tc_ld_32x16(t_row + 16, zx);
          tc_ld_32x16(t_row + kUT + 16, za);
        }
        {
          const uint4 c0 = lds_piece(tile_c_s + row_off, 2 * half), c1 = lds_piece(tile_c_s + row_off, 2 * half + 1);
          c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w;
          c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
        }
        tc_wait_ld();
        if (half == 1) {
          // the accumulator set has been read: it may be overwritten
          tc_fence_before();
          __syncwarp();
          if (lane == 0 && ok) mbar_arrive(bar_acc_empty(as));
          // ... and so has the conv tile: the next unit's is fetched into it (the generic-proxy
          // accesses of every lane are ordered before the copy engine's write)
          fence_proxy_async();
          __syncwarp();
          if constexpr (kConv) {
            if (lane == 0) mbar_arrive(bar_cfree);   // the conv warps may write the next unit's tile
          } else if (lane == 0 && t + 1 < n_my) {
            mbar_expect_tx(bar_ct(warp), kSubBytes);
            tma_load_3d(tile_c_s, &map_ct, chan0(nxt), nxt.tt * kUT + tq * kSub, nxt.b, bar_ct(warp));
          }
        }
        const uint32_t rs = (resets >> (half * 16)) & 0xffffu;
        const uint32_t inv = (invalid >> (half * 16)) & 0xffffu;
        if ((rs | inv) == 0u)
          gates_16<false, kMath>(zx, za, c, bx2, ba2, hbx2, m8sp2, rs, inv, a_pk + half * 8,
                                 x_pk + half * 8, P, H, s_lut);
        else
          gates_16<true, kMath>(zx, za, c, bx2, ba2, hbx2, m8sp2, rs, inv, a_pk + half * 8,
                                x_pk + half * 8, P, H, s_lut);
        if (half == 0) {
          // the previous unit's output tile must have been read by its store before the buffer is
          // written again; then the other branch's tile of this unit is fetched into it
          if (lane == 0) {
            bulk_wait_read();
            if constexpr (kJoin != 0) {
              mbar_expect_tx(bar_yt(warp), kSubBytes);
              tma_load_3d(tile_y_s, &map_yt, e0, tok0, b, bar_yt(warp));
            }
          }
        }
      }
      if (t + 1 < n_my) load_consts(nxt);
      if (t + 1 < n_my) reset_next = lane_reset(nxt);

      // The incoming state is normally known before the tile's own map is (the predecessor's
      // inclusive record was there at the start of the unit): then the quarters need one barrier,
      // to see each other's maps, and nothing waits for the record of this tile to be published.
      if (tq == 3) {
        if (tt > 0) {
          bool all = __all_sync(0xffffffffu, (pre >> 32) == 1ull);
          if (!all) {
            // the predecessor's CTA runs a little behind: ask once more before taking the long way
            pre = ld_relaxed_u64(incl + (rec - (int64_t)per_tt * 4) * kSub + lane);
            all = __all_sync(0xffffffffu, (pre >> 32) == 1ull);
          }
          if (all) {
            hin_pref = __uint_as_float((uint32_t)pre);
            have_hin = true;
          }
        }
        if (have_hin) s_hin[lane] = hin_pref;
        if (lane == 0) *s_known = have_hin ? 1 : 0;
      }
      if (tq < 3) s_qmap[tq * 32 + lane] = make_float2(P, H);   // the last quarter keeps its own
      named_bar_sync(set_id, 128);
      const bool known = *s_known != 0;

      // ---- the last token quarter: the tile's map, the incoming state, the records ---------------
      if (tq == 3) {
        float Pt = 1.0f, Ht = 0.0f;
#pragma unroll
        for (int qq = 0; qq < 3; ++qq) {
          const float2 m = s_qmap[qq * 32 + lane];
          Ht = fmaf(m.x, Ht, m.y);
          Pt *= m.x;
        }
        Ht = fmaf(P, Ht, H);
        Pt *= P;
        float hin = hin_pref;
        if (!known) {
          // Decoupled look-back, one channel per lane.  With use_agg (fewer chains than CTAs: the
          // earlier tiles of this chain are in flight on other SMs) the tile's own map is published
          // first, and maps of earlier tiles are composed until a tile with a known state is met;
          // otherwise only the predecessor's state is waited for (it was dealt out a round earlier).
          if (use_agg && RGK_IN_RANGE(rec * kSub + lane, n_words, &hdr->status)) {
            st_relaxed_u64(agg + (rec * kSub + lane) * 2, kToken | (unsigned long long)__float_as_uint(Pt));
            st_relaxed_u64(agg + (rec * kSub + lane) * 2 + 1, kToken | (unsigned long long)__float_as_uint(Ht));
          }
          bool timed_out = false;
          if (ok) hin = look_back(agg, incl, h0, rec, tt, per_tt, b, E, e0 + lane, lane, use_agg, &timed_out,
                                 n_words, n_state, &hdr->status);
          __syncwarp();
          if (__any_sync(0xffffffffu, timed_out)) {
            if (lane == 0) atomicExch(&hdr->status, kStatusTimeout);
            hin = 0.0f;
          }
          if (!ok) hin = 0.0f;
          s_hin[lane] = hin;
        }
        const float h_end = fmaf(Pt, hin, Ht);
        if (RGK_IN_RANGE(rec * kSub + lane, n_words, &hdr->status))
          st_relaxed_u64(incl + rec * kSub + lane, kToken | (unsigned long long)__float_as_uint(h_end));
        if (h_last != nullptr && tt == tiles_t - 1 &&
            RGK_IN_RANGE((int64_t)b * E + e0 + lane, n_state, &hdr->status))
          h_last[(int64_t)b * E + e0 + lane] = h_end;
      }
      if (!known) named_bar_sync(set_id, 128);

      // ---- replay with the true incoming state, join, output tile ---------------------------------
      float h = s_hin[lane];
      for (int qq = 0; qq < tq; ++qq) {
        const float2 m = s_qmap[qq * 32 + lane];
        h = fmaf(m.x, h, m.y);
      }
      if constexpr (kJoin != 0) {
        if (ok) ok = mbar_wait(bar_yt(warp), t & 1, s_abort);
        transpose_tile(tile_y_s + row_off, tile_y_s + st_off);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint32_t z[4] = {0u, 0u, 0u, 0u}, o[4];
        if constexpr (kJoin != 0) {
          const uint4 zv = lds_piece(tile_y_s + row_off, k);
          z[0] = zv.x; z[1] = zv.y; z[2] = zv.z; z[3] = zv.w;
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint32_t a2 = a_pk[4 * k + w], x2 = x_pk[4 * k + w];
          h = fmaf(bf16_lo(a2), h, bf16_lo(x2));
          const float y0 = h;
          h = fmaf(bf16_hi(a2), h, bf16_hi(x2));
          uint32_t y2 = pack_bf16x2(y0, h);
          if constexpr (kJoin == 1) y2 = join_gelu2<kMath>(y2, z[w]);
          else if constexpr (kJoin == 2) y2 = bmul2(y2, z[w]);
          o[w] = y2;
        }
        sts_piece(tile_y_s + row_off, k, make_uint4(o[0], o[1], o[2], o[3]));
      }
      __syncwarp();
      transpose_tile(tile_y_s + row_off, tile_y_s + st_off);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        tma_store_3d(&map_ot, e0, tok0, b, tile_y_s);
        bulk_commit();
      }
      cur = nxt;
    }
    if (lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *s_abort) atomicExch(&hdr->status, kStatusTimeout);
  if (warp == kEpi + 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512)
                 : "memory");
  }
}

// -8 softplus(a_param), rounded as the reference rounds its factors, one value per channel.
__global__ void m8sp_chan_kernel(const __nv_bfloat16* __restrict__ a_param, int E,
                                 __nv_bfloat16* __restrict__ m8sp) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < E) {
    const float s = round_bf16(softplus_(__bfloat162float(a_param[e])));
    // clamped to the range of the kernel's table of exp(log_a): beyond it a = exp(log_a) is 0 in
    // float32 either way (the gate would have to be below 0.7 at softplus(a_param) above 16)
    m8sp[e] = __float2bfloat16_rn(fmaxf(-8.0f * s, kLogAFloor));
  }
}

// Tensor map of a row-major bfloat16 matrix [rows, cols] with boxes of box_rows x box_cols.


// Tensor map of bfloat16 activations [B, T, E] with boxes of box_rows tokens x box_cols channels of
// one sequence: rows past the end of a sequence read as zero and are dropped from stores.


struct ChanLayout {
  int64_t n_units, n_rec;
  size_t m8sp_off, agg_off, incl_off, total;
};

ChanLayout chan_layout(int64_t B, int64_t T, int64_t E) {
  ChanLayout L;
  const int64_t groups = E / kUC;
  L.n_units = ((T + kUT - 1) / kUT) * B * groups;
  L.n_rec = L.n_units * 4;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  L.incl_off = sizeof(WsHeader);
  L.agg_off = up(L.incl_off + (size_t)L.n_rec * kSub * sizeof(unsigned long long));
  L.m8sp_off = up(L.agg_off + (size_t)L.n_rec * kSub * 2 * sizeof(unsigned long long));
  L.total = up(L.m8sp_off + (size_t)E * 2);
  return L;
}

// The kernel needs more dynamic shared memory than the default limit: the attribute is a property
// of the function on ONE device, so it is set (and the SM count read) once per device.
template <int kMath, bool kConv>
cudaError_t chan_set_smem() {
  cudaError_t e;
  if ((e = cudaFuncSetAttribute(rglru_chan_kernel<0, kMath, kConv>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(rglru_chan_kernel<1, kMath, kConv>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem)) != cudaSuccess) return e;
  return cudaFuncSetAttribute(rglru_chan_kernel<2, kMath, kConv>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
}

cudaError_t chan_device_setup(int* num_sms) {
  static PerDeviceOnce once;
  return once.run([] {
    cudaError_t e;
    if ((e = chan_set_smem<kMathExact, false>()) != cudaSuccess) return e;
    if ((e = chan_set_smem<kMathFast, false>()) != cudaSuccess) return e;
    if ((e = chan_set_smem<kMathExact, true>()) != cudaSuccess) return e;
    return chan_set_smem<kMathFast, true>();
  }, num_sms);
}

}  // namespace

bool rglru_chan_supported(int dtype, int bw, int64_t B, int64_t T) {
  return dtype == 1 && bw == kHW && B >= 1 && T >= 1 && B * T < ((int64_t)1 << 31);
}

size_t rglru_chan_workspace_bytes(int64_t B, int64_t T, int64_t E) {
  if (T < 1) return 0;
  return chan_layout(B, T, E).total;
}

cudaError_t launch_rglru_chan(const void* c, const void* pos, int pos64, const void* a_param,
                              const void* bx, const void* ba, const void* packed_w, const float* h0,
                              const void* yb, int y_activated, int64_t B, int64_t T, int H,
                              void* out, float* h_last, void* ws, int math, cudaStream_t s,
                              const void* conv_w, const void* conv_b) {
  using T_ = __nv_bfloat16;
  const bool conv = conv_w != nullptr;       // `c` is then the block input, the kernel convolves it
  const int E = H * kHW;
  const ChanLayout L = chan_layout(B, T, E);
  char* base = static_cast<char*>(ws);
  int num_sms = 0;
  cudaError_t err = chan_device_setup(&num_sms);
  if (err != cudaSuccess) return err;
  const int groups = 2 * H;
  const int n_units = (int)L.n_units;
  const int grid = n_units < num_sms ? n_units : num_sms;   // all CTAs resident: look-back may spin
  // With fewer units per time tile than CTAs, consecutive tiles of a chain are in flight at once
  // and carries are resolved from published maps; otherwise a tile's predecessor was dealt out a
  // round earlier and only its state is ever waited for.
  const int use_agg = (int64_t)B * groups < grid ? 1 : 0;
  // state words (and map words, where used) start without their token; the status word before
  // them belongs to the caller
  err = cudaMemsetAsync(base + sizeof(int), 0, (use_agg ? L.m8sp_off : L.agg_off) - sizeof(int), s);
  if (err != cudaSuccess) return err;
  T_* m8sp = reinterpret_cast<T_*>(base + L.m8sp_off);
  m8sp_chan_kernel<<<(E + 255) / 256, 256, 0, s>>>((const T_*)a_param, E, m8sp);
  if ((err = cudaGetLastError()) != cudaSuccess) return err;

  CUtensorMap map_c, map_w, map_ct, map_yt, map_ot;
  const uint64_t Bu = (uint64_t)B, Tu = (uint64_t)T, Eu = (uint64_t)E;
  if (!(conv ? tensor_map_bte(&map_c, c, Bu, Tu, Eu, kXRows, kKB, false)
             : tensor_map_bte(&map_c, c, Bu, Tu, Eu, kUT, kKB, true)) ||
      !tensor_map_2d(&map_w, packed_w, (uint64_t)H * 4 * kUC, kHW, 2 * kUC, kKB, true) ||
      !tensor_map_bte_sw64(&map_ct, c, Bu, Tu, Eu, kSub, kSub) ||
      !tensor_map_bte_sw64(&map_ot, out, Bu, Tu, Eu, kSub, kSub) ||
      !tensor_map_bte_sw64(&map_yt, yb != nullptr ? yb : out, Bu, Tu, Eu, kSub, kSub))
    return cudaErrorInvalidValue;
#define RGK_CHAN_C(J, M, C, THREADS)                                                             \
  rglru_chan_kernel<J, M, C><<<grid, THREADS, kSmem, s>>>(                                       \
      map_c, map_w, map_ct, map_yt, map_ot, pos, pos64, (const T_*)bx, (const T_*)ba, m8sp, h0,  \
      (int)B, (int)T, E, groups, n_units, h_last, reinterpret_cast<WsHeader*>(base),             \
      reinterpret_cast<unsigned long long*>(base + L.agg_off),                                   \
      reinterpret_cast<unsigned long long*>(base + L.incl_off), use_agg, (const T_*)conv_w,      \
      (const T_*)conv_b)
#define RGK_CHAN(J, M)                                                                           \
  do { if (conv) RGK_CHAN_C(J, M, true, kThreadsConv); else RGK_CHAN_C(J, M, false, kThreads); } while (0)
#define RGK_CHAN_J(M)                                                                            \
  if (join == 0) RGK_CHAN(0, M); else if (join == 1) RGK_CHAN(1, M); else RGK_CHAN(2, M)
  const int join = yb == nullptr ? 0 : (y_activated ? 2 : 1);
  switch (math) {
    case kMathExact: RGK_CHAN_J(kMathExact); break;
    case kMathFast: RGK_CHAN_J(kMathFast); break;
    default: return cudaErrorInvalidValue;
  }
#undef RGK_CHAN_J
#undef RGK_CHAN
#undef RGK_CHAN_C
  return cudaGetLastError();
}

}  // namespace rgk
