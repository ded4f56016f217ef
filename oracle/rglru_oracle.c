/*
 * CPU oracle for the RG-LRU + Conv1D path of recurrentgemma's torch implementation.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are compared with
 * (and the timed CPU baseline of the benchmark).  Nothing in the shipped package may call it.
 *
 * It restates, in plain C, what the reference computes in
 *   recurrentgemma/torch/layers.py   (BlockDiagonalLinear 127-137, rnn_scan 140-191,
 *                                     RGLRU.forward 313-365, Conv1D.forward 447-529 and its
 *                                     helpers 531-636)
 *   recurrentgemma/torch/modules.py  (gelu 289-291, RecurrentBlock.forward 605-655)
 * Parity is pinned by execution: tests/golden/ holds outputs of the reference itself on seeded
 * inputs (made by tests/golden/make_golden.py) and tests/test_oracle_golden.py checks this file
 * against every one of them.
 *
 * Numeric model.  All arrays are float32.  `dt` selects the arithmetic the reference would have
 * run in: RGO_F32 keeps float32 everywhere; RGO_BF16 rounds the result of every tensor-level
 * operation of the reference to bfloat16 (round to nearest even), which is what torch does when
 * its tensors are bfloat16 (each elementwise kernel computes in float and stores bfloat16).
 * Inputs must then already be bfloat16-representable.  The recurrence state is float32 in both
 * modes (layers.py:146, 176, 184-189).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define RGO_F32 0
#define RGO_BF16 1

#if defined(__GNUC__)
#define RGO_API __attribute__((visibility("default")))
#else
#define RGO_API
#endif

/* Round a float to the nearest bfloat16 (ties to even) and return it as a float. */
static inline float rbf(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) { /* NaN: keep it a NaN */
    u |= 0x00400000u;
    u &= 0xffff0000u;
  } else {
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
  }
  memcpy(&v, &u, 4);
  return v;
}

static inline float rnd(float v, int dt) { return dt == RGO_BF16 ? rbf(v) : v; }

static inline float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

/* torch.nn.functional.softplus with its defaults (beta 1, threshold 20). */
static inline float softplusf_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

/* gelu(approximate="tanh"), modules.py:289-291. */
static inline float gelu_tanhf_(float z) {
  const float k0 = 0.7978845608028654f; /* sqrt(2/pi) */
  const float k1 = 0.044715f;
  float inner = k0 * (z + k1 * z * z * z);
  return 0.5f * z * (1.0f + tanhf(inner));
}

RGO_API int rgo_version(void) { return 5; }

/* OpenMP thread count of the parallel loops below.  A launcher may have exported OMP_NUM_THREADS=1
 * to every process it starts (torch.distributed.run does), so a timed baseline sets the count
 * itself and reports what the runtime then gives.  Without OpenMP both return 1. */
#ifdef _OPENMP
#include <omp.h>
RGO_API int rgo_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}
RGO_API int rgo_max_threads(void) { return omp_get_max_threads(); }
#else
RGO_API int rgo_set_threads(int n) { (void)n; return 1; }
RGO_API int rgo_max_threads(void) { return 1; }
#endif

/* ---------------------------------------------------------------------------------------------
 * BlockDiagonalLinear.forward, layers.py:127-137.
 *   x [M, H*bw], w [H, bw(in), bw(out)], b [H, bw]  ->  out [M, H*bw]
 * The contraction accumulates in float32 and is stored in the tensor dtype; the bias add is a
 * second tensor operation (layers.py:134), hence a second rounding in bfloat16 mode.
 * ------------------------------------------------------------------------------------------- */
RGO_API void rgo_blockdiag_linear(const float* x, const float* w, const float* b, int64_t M,
                                  int H, int bw, int dt, float* out) {
  const int64_t E = (int64_t)H * bw;
  enum { RB = 8 }; /* rows that share one pass over a head's weights */
  const int64_t n_rb = (M + RB - 1) / RB;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t rb = 0; rb < n_rb; ++rb) {
    for (int h = 0; h < H; ++h) {
      const int64_t m0 = rb * RB;
      const int rows = (int)((M - m0) < RB ? (M - m0) : RB);
      float* acc = (float*)malloc(sizeof(float) * (size_t)RB * (size_t)bw);
      for (int i = 0; i < RB * bw; ++i) acc[i] = 0.0f;
      const float* wh = w + (int64_t)h * bw * bw;
      for (int i = 0; i < bw; ++i) {
        const float* wr = wh + (int64_t)i * bw;
        for (int r = 0; r < rows; ++r) {
          const float xi = x[(m0 + r) * E + (int64_t)h * bw + i];
          float* ar = acc + (size_t)r * bw;
          for (int j = 0; j < bw; ++j) ar[j] += xi * wr[j];
        }
      }
      const float* bh = b + (int64_t)h * bw;
      for (int r = 0; r < rows; ++r) {
        float* o = out + (m0 + r) * E + (int64_t)h * bw;
        const float* ar = acc + (size_t)r * bw;
        for (int j = 0; j < bw; ++j) o[j] = rnd(rnd(ar[j], dt) + bh[j], dt);
      }
      free(acc);
    }
  }
}

/* ---------------------------------------------------------------------------------------------
 * nn.Linear as used by RecurrentBlock (modules.py:531-548): out = x @ weight^T + bias with
 * weight [N, K].  One rounding of the float32 accumulator plus bias.
 * ------------------------------------------------------------------------------------------- */
RGO_API void rgo_linear(const float* x, const float* weight, const float* bias, int64_t M, int K,
                        int N, int dt, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    const float* xr = x + m * K;
    for (int n = 0; n < N; ++n) {
      const float* wr = weight + (int64_t)n * K;
      float acc = 0.0f;
#pragma omp simd reduction(+ : acc)
      for (int k = 0; k < K; ++k) acc += xr[k] * wr[k];
      out[m * N + n] = rnd(acc + (bias ? bias[n] : 0.0f), dt);
    }
  }
}

/* ---------------------------------------------------------------------------------------------
 * Conv1D.forward without a cache (prefill / training form), layers.py:476-529.
 *   x [B,T,E], segment_pos [B,T], w [W,E], b [E]  ->  out [B,T,E], cache [B,W-1,E] (may be NULL)
 * For shift s = 0 .. min(W,T)-1 the reference multiplies the window x[:, 0:T-s] IN PLACE by a
 * 0/1 document mask (layers.py:497-508) that is 0 where any of the next s positions starts a
 * document (segment_pos == 0, layers.py:598-607), then accumulates window * w[W-1-s] shifted
 * right by s (layers.py:510-517).  The masks are nested, so the in-place products equal the
 * product over k = t-s+1 .. t of (segment_pos[k] != 0) for the tap that reaches output t.
 * The returned cache is the last W-1 rows of that mutated input, left padded with zeros
 * (layers.py:526-527, 624-636): row T-1-j has been multiplied by the masks of shifts 1..j only.
 * ------------------------------------------------------------------------------------------- */
RGO_API void rgo_conv1d_prefill(const float* x, const int64_t* segment_pos, const float* w,
                                const float* b, int B, int T, int E, int W, int dt, float* out,
                                float* cache) {
  const int nshift = W < T ? W : T;
#pragma omp parallel for collapse(2) schedule(static)
  for (int bi = 0; bi < B; ++bi) {
    for (int t = 0; t < T; ++t) {
      const int64_t* pos = segment_pos + (int64_t)bi * T;
      float* o = out + ((int64_t)bi * T + t) * E;
      /* keep[s] = 1 while no document start lies in (t-s, t]; -1 when tap s falls into the
         left zero padding (layers.py:510, 609-622). */
      int keep[64];
      int alive = 1;
      for (int s = 0; s < nshift && s < 64; ++s) {
        if (s > t) {
          keep[s] = -1;
          continue;
        }
        if (s > 0 && pos[t - s + 1] == 0) alive = 0;
        keep[s] = alive;
      }
      for (int e = 0; e < E; ++e) {
        float acc = 0.0f;
        for (int s = 0; s < nshift; ++s) {
          float xv;
          if (keep[s] < 0) {
            xv = 0.0f;
          } else {
            xv = x[((int64_t)bi * T + (t - s)) * E + e];
            if (!keep[s]) xv = xv * 0.0f;
          }
          const float prod = rnd(xv * w[(int64_t)(W - 1 - s) * E + e], dt);
          acc = (s == 0) ? prod : rnd(acc + prod, dt);
        }
        o[e] = rnd(acc + b[e], dt);
      }
    }
  }
  if (cache) {
    for (int bi = 0; bi < B; ++bi) {
      const int64_t* pos = segment_pos + (int64_t)bi * T;
      for (int i = 0; i < W - 1; ++i) {
        const int t = T - (W - 1) + i;
        float* c = cache + ((int64_t)bi * (W - 1) + i) * E;
        if (t < 0) {
          for (int e = 0; e < E; ++e) c[e] = 0.0f;
          continue;
        }
        /* Row t was inside the window of shift s iff t <= T-1-s, and was then multiplied by
           prod_{k=1..s} (pos[t+k] != 0), for s < nshift. */
        int alive = 1;
        for (int s = 1; s < nshift && t + s <= T - 1; ++s)
          if (pos[t + s] == 0) alive = 0;
        for (int e = 0; e < E; ++e) {
          const float xv = x[((int64_t)bi * T + t) * E + e];
          c[e] = alive ? xv : xv * 0.0f;
        }
      }
    }
  }
}

/* ---------------------------------------------------------------------------------------------
 * Conv1D.forward with a cache (single-token decode), layers.py:469-474, 487-529, 531-550.
 *   x [B,E] (the one new token), cache [B,W-1,E]  ->  out [B,E], new_cache [B,W-1,E]
 * No document masking in this mode (layers.py:499).  Taps are accumulated newest first.
 * ------------------------------------------------------------------------------------------- */
RGO_API void rgo_conv1d_decode(const float* x, const float* cache, const float* w, const float* b,
                               int B, int E, int W, int dt, float* out, float* new_cache) {
#pragma omp parallel for schedule(static)
  for (int bi = 0; bi < B; ++bi) {
    for (int e = 0; e < E; ++e) {
      float acc = 0.0f;
      for (int s = 0; s < W; ++s) {
        const int idx = W - 1 - s; /* position inside concat([cache, x]) */
        const float xv = (idx == W - 1) ? x[(int64_t)bi * E + e]
                                        : cache[((int64_t)bi * (W - 1) + idx) * E + e];
        const float prod = rnd(xv * w[(int64_t)idx * E + e], dt);
        acc = (s == 0) ? prod : rnd(acc + prod, dt);
      }
      out[(int64_t)bi * E + e] = rnd(acc + b[e], dt);
    }
    if (new_cache) {
      for (int i = 0; i < W - 1; ++i)
        for (int e = 0; e < E; ++e)
          new_cache[((int64_t)bi * (W - 1) + i) * E + e] =
              (i + 1 == W - 1) ? x[(int64_t)bi * E + e]
                               : cache[((int64_t)bi * (W - 1) + i + 1) * E + e];
    }
  }
}

/* ---------------------------------------------------------------------------------------------
 * rnn_scan, layers.py:140-191.
 *   x, a [B,T,E] (tensor dtype), reset [B,T] (0/1), h0 [B,E] float32 or NULL
 *   ->  y [B,T,E] (tensor dtype), h_last [B,E] float32
 * `a` is first multiplied by !reset (layers.py:168).  T == 1 takes the sampling branch
 * (layers.py:170-177): without h0 the output is x itself; with h0 the new state is the
 * unrounded float32 value.
 * ------------------------------------------------------------------------------------------- */
RGO_API void rgo_rnn_scan(const float* x, const float* a, const uint8_t* reset, const float* h0,
                          int B, int T, int E, int dt, float* y, float* h_last) {
  if (T == 1 && !h0) {
    for (int64_t i = 0; i < (int64_t)B * E; ++i) {
      y[i] = x[i];
      if (h_last) h_last[i] = x[i];
    }
    return;
  }
#pragma omp parallel for collapse(2) schedule(static)
  for (int bi = 0; bi < B; ++bi) {
    for (int e0 = 0; e0 < E; e0 += 64) {
      const int e1 = e0 + 64 < E ? e0 + 64 : E;
      float h[64];
      for (int e = e0; e < e1; ++e) h[e - e0] = h0 ? h0[(int64_t)bi * E + e] : 0.0f;
      for (int t = 0; t < T; ++t) {
        const int64_t row = ((int64_t)bi * T + t) * E;
        const float keep = reset[(int64_t)bi * T + t] ? 0.0f : 1.0f;
        for (int e = e0; e < e1; ++e) {
          const float at = a[row + e] * keep; /* exact: times 0 or 1 */
          h[e - e0] = at * h[e - e0] + x[row + e];
          y[row + e] = rnd(h[e - e0], dt);
        }
      }
      if (h_last)
        for (int e = e0; e < e1; ++e) h_last[(int64_t)bi * E + e] = h[e - e0];
    }
  }
}

/* ---------------------------------------------------------------------------------------------
 * The gate / normalisation arithmetic of RGLRU.forward, layers.py:338-353, for one element.
 * zx, za are the outputs of the two BlockDiagonalLinear layers; sp = softplus(a_param).
 * Writes a (before the reset mask) and the normalised input.
 * ------------------------------------------------------------------------------------------- */
static inline void rglru_pointwise(float xv, float zx, float za, float sp, int is_reset, int dt,
                                   float* a_out, float* xn_out) {
  const float gate_x = rnd(sigmoidf_(zx), dt);
  const float gate_a = rnd(sigmoidf_(za), dt);
  const float log_a = rnd(rnd(-8.0f * gate_a, dt) * sp, dt);
  const float a = rnd(expf(log_a), dt);
  const float a_square = rnd(expf(rnd(2.0f * log_a, dt)), dt);
  const float gated_x = rnd(xv * gate_x, dt);
  float mult = rnd(sqrtf(rnd(1.0f - a_square, dt)), dt);
  if (is_reset) mult = 1.0f;
  *a_out = a;
  *xn_out = rnd(gated_x * mult, dt);
}

/* ---------------------------------------------------------------------------------------------
 * RGLRU.forward, layers.py:313-365.
 *   x [B,T,E], segment_pos [B,T], a_param [E], gates w [H,bw,bw] / b [H,bw], h0 [B,E] or NULL
 *   ->  y [B,T,E], h_last [B,E] float32.   scratch: 4 * B*T*E floats are allocated inside.
 * Returns 0, or -1 if the scratch allocation failed.
 * ------------------------------------------------------------------------------------------- */
RGO_API int rgo_rglru(const float* x, const int64_t* segment_pos, const float* a_param,
                      const float* wx, const float* bx, const float* wa, const float* ba,
                      const float* h0, int B, int T, int E, int H, int dt, float* y,
                      float* h_last) {
  const int64_t M = (int64_t)B * T, N = M * E;
  const int bw = E / H;
  float* zx = (float*)malloc(sizeof(float) * (size_t)N);
  float* za = (float*)malloc(sizeof(float) * (size_t)N);
  uint8_t* reset = (uint8_t*)malloc((size_t)M);
  float* sp = (float*)malloc(sizeof(float) * (size_t)E);
  if (!zx || !za || !reset || !sp) {
    free(zx); free(za); free(reset); free(sp);
    return -1;
  }
  rgo_blockdiag_linear(x, wx, bx, M, H, bw, dt, zx);
  rgo_blockdiag_linear(x, wa, ba, M, H, bw, dt, za);
  for (int e = 0; e < E; ++e) sp[e] = rnd(softplusf_(a_param[e]), dt);
  for (int64_t m = 0; m < M; ++m) reset[m] = segment_pos[m] == 0;
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    for (int e = 0; e < E; ++e) {
      float a, xn;
      rglru_pointwise(x[m * E + e], zx[m * E + e], za[m * E + e], sp[e], reset[m], dt, &a, &xn);
      za[m * E + e] = a;  /* reuse the buffers: za <- a, zx <- normalised x */
      zx[m * E + e] = xn;
    }
  }
  rgo_rnn_scan(zx, za, reset, h0, B, T, E, dt, y, h_last);
  free(zx); free(za); free(reset); free(sp);
  return 0;
}

/* y * gelu(y_branch): modules.py:627-628 and 646.  Both factors are tensors of the block dtype. */
RGO_API void rgo_gelu_mul(const float* y, const float* y_branch, int64_t n, int dt, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
    out[i] = rnd(y[i] * rnd(gelu_tanhf_(y_branch[i]), dt), dt);
}

/* ---------------------------------------------------------------------------------------------
 * The RG-LRU + Conv1D sub-path of RecurrentBlock.forward (modules.py:631-646) given the two
 * projected branches:  out = RGLRU(Conv1D(xb)) * gelu(yb).
 *   prefill: conv_cache_in == NULL, T >= 1;  decode: conv_cache_in != NULL, T == 1.
 * Outputs: out [B,T,E], h_last [B,E], conv_cache_out [B,W-1,E].
 * ------------------------------------------------------------------------------------------- */
RGO_API int rgo_recurrent_path(const float* xb, const float* yb, const int64_t* segment_pos,
                               const float* conv_w, const float* conv_b, const float* a_param,
                               const float* wx, const float* bx, const float* wa, const float* ba,
                               const float* h0, const float* conv_cache_in, int B, int T, int E,
                               int H, int W, int dt, float* out, float* h_last,
                               float* conv_cache_out) {
  const int64_t N = (int64_t)B * T * E;
  float* c = (float*)malloc(sizeof(float) * (size_t)N);
  float* y = (float*)malloc(sizeof(float) * (size_t)N);
  if (!c || !y) {
    free(c); free(y);
    return -1;
  }
  if (conv_cache_in) {
    if (T != 1) { free(c); free(y); return -2; } /* layers.py:549 */
    rgo_conv1d_decode(xb, conv_cache_in, conv_w, conv_b, B, E, W, dt, c, conv_cache_out);
  } else {
    rgo_conv1d_prefill(xb, segment_pos, conv_w, conv_b, B, T, E, W, dt, c, conv_cache_out);
  }
  int rc = rgo_rglru(c, segment_pos, a_param, wx, bx, wa, ba, h0, B, T, E, H, dt, y, h_last);
  if (rc == 0) rgo_gelu_mul(y, yb, N, dt, out);
  free(c); free(y);
  return rc;
}

/* ---------------------------------------------------------------------------------------------
 * RecurrentBlock.forward, modules.py:605-655: the sub-path above between linear_x / linear_y
 * and linear_out.  x [B,T,D]; linear weights in nn.Linear layout [out,in].
 * ------------------------------------------------------------------------------------------- */
RGO_API int rgo_recurrent_block(const float* x, const int64_t* segment_pos, const float* wy,
                                const float* by, const float* wxl, const float* bxl,
                                const float* wout, const float* bout, const float* conv_w,
                                const float* conv_b, const float* a_param, const float* gwx,
                                const float* gbx, const float* gwa, const float* gba,
                                const float* h0, const float* conv_cache_in, int B, int T, int D,
                                int E, int H, int W, int dt, float* out, float* h_last,
                                float* conv_cache_out) {
  const int64_t M = (int64_t)B * T;
  float* xb = (float*)malloc(sizeof(float) * (size_t)(M * E));
  float* yb = (float*)malloc(sizeof(float) * (size_t)(M * E));
  float* z = (float*)malloc(sizeof(float) * (size_t)(M * E));
  if (!xb || !yb || !z) {
    free(xb); free(yb); free(z);
    return -1;
  }
  rgo_linear(x, wy, by, M, D, E, dt, yb);
  rgo_linear(x, wxl, bxl, M, D, E, dt, xb);
  int rc = rgo_recurrent_path(xb, yb, segment_pos, conv_w, conv_b, a_param, gwx, gbx, gwa, gba,
                              h0, conv_cache_in, B, T, E, H, W, dt, z, h_last, conv_cache_out);
  if (rc == 0) rgo_linear(z, wout, bout, M, E, D, dt, out);
  free(xb); free(yb); free(z);
  return rc;
}

/* ---------------------------------------------------------------------------------------------
 * RMSNorm.forward, layers.py:65-73:
 *   var = mean(square(x), -1);  normed = x * rsqrt(var + eps);  out = normed * (scale + 1)
 * x [M, D], scale [D].  Each tensor operation rounds in bfloat16 mode: the squares, the mean (one
 * rounding of the float32 sum divided by D), var + eps, the reciprocal square root, the product
 * with it, scale + 1 and the final product.
 * ------------------------------------------------------------------------------------------- */
RGO_API void rgo_rmsnorm(const float* x, const float* scale, int64_t M, int D, float eps, int dt,
                         float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    const float* xr = x + m * D;
    float sum = 0.0f;
    for (int k = 0; k < D; ++k) sum += rnd(xr[k] * xr[k], dt);
    const float var = rnd(sum / (float)D, dt);
    const float r = rnd(1.0f / sqrtf(rnd(var + eps, dt)), dt);
    for (int k = 0; k < D; ++k)
      out[m * D + k] = rnd(rnd(xr[k] * r, dt) * rnd(scale[k] + 1.0f, dt), dt);
  }
}

/* ---------------------------------------------------------------------------------------------
 * The temporal half of ResidualBlock.forward for a recurrent block, modules.py:897-902:
 *   residual = recurrent_block(temporal_pre_norm(x)) + x
 * ------------------------------------------------------------------------------------------- */
RGO_API int rgo_residual_temporal(const float* x, const int64_t* segment_pos,
                                  const float* norm_scale, float eps, const float* wy,
                                  const float* by, const float* wxl, const float* bxl,
                                  const float* wout, const float* bout, const float* conv_w,
                                  const float* conv_b, const float* a_param, const float* gwx,
                                  const float* gbx, const float* gwa, const float* gba,
                                  const float* h0, const float* conv_cache_in, int B, int T, int D,
                                  int E, int H, int W, int dt, float* out, float* h_last,
                                  float* conv_cache_out) {
  const int64_t M = (int64_t)B * T;
  float* xn = (float*)malloc(sizeof(float) * (size_t)(M * D));
  if (!xn) return -1;
  rgo_rmsnorm(x, norm_scale, M, D, eps, dt, xn);
  int rc = rgo_recurrent_block(xn, segment_pos, wy, by, wxl, bxl, wout, bout, conv_w, conv_b,
                               a_param, gwx, gbx, gwa, gba, h0, conv_cache_in, B, T, D, E, H, W,
                               dt, out, h_last, conv_cache_out);
  if (rc == 0)
    for (int64_t i = 0; i < M * D; ++i) out[i] = rnd(out[i] + x[i], dt);
  free(xn);
  return rc;
}

/* ---------------------------------------------------------------------------------------------
 * MLPBlock.forward, modules.py:740-752 with Einsum.forward, layers.py:700-703:
 *   out_c = einsum("...td,cdD->c...tD", x, w)[c] + b[c]   (c = 0, 1; two tensor operations, so the
 *           contraction is rounded before the bias is added and the sum is rounded again)
 *   act   = gelu_tanh(out_0) * out_1
 *   y     = ffw_down(act)  (nn.Linear: one rounding of accumulator + bias)
 * x [M, D], w_up [2, D, X] (in, out), b_up [2, X], w_down [D, X] (nn.Linear layout), b_down [D].
 * ------------------------------------------------------------------------------------------- */
RGO_API int rgo_mlp(const float* x, const float* w_up, const float* b_up, const float* w_down,
                    const float* b_down, int64_t M, int D, int X, int dt, float* out) {
  float* act = (float*)malloc(sizeof(float) * (size_t)(M * X));
  if (!act) return -1;
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    float* acc = (float*)malloc(sizeof(float) * (size_t)(2 * X));
    for (int j = 0; j < 2 * X; ++j) acc[j] = 0.0f;
    const float* xr = x + m * D;
    for (int k = 0; k < D; ++k) {
      const float xv = xr[k];
      const float* w0 = w_up + (int64_t)k * X;
      const float* w1 = w_up + ((int64_t)D + k) * X;
      for (int j = 0; j < X; ++j) { acc[j] += xv * w0[j]; acc[X + j] += xv * w1[j]; }
    }
    for (int j = 0; j < X; ++j) {
      const float o0 = rnd(rnd(acc[j], dt) + b_up[j], dt);
      const float o1 = rnd(rnd(acc[X + j], dt) + b_up[X + j], dt);
      act[m * X + j] = rnd(rnd(gelu_tanhf_(o0), dt) * o1, dt);
    }
    free(acc);
  }
  rgo_linear(act, w_down, b_down, M, X, D, dt, out);
  free(act);
  return 0;
}

/* ---------------------------------------------------------------------------------------------
 * The channel half of ResidualBlock.forward, modules.py:904-908:
 *   out = mlp_block(channel_pre_norm(residual)) + residual
 * ------------------------------------------------------------------------------------------- */
RGO_API int rgo_residual_channel(const float* residual, const float* norm_scale, float eps,
                                 const float* w_up, const float* b_up, const float* w_down,
                                 const float* b_down, int64_t M, int D, int X, int dt,
                                 float* out) {
  float* xn = (float*)malloc(sizeof(float) * (size_t)(M * D));
  if (!xn) return -1;
  rgo_rmsnorm(residual, norm_scale, M, D, eps, dt, xn);
  int rc = rgo_mlp(xn, w_up, b_up, w_down, b_down, M, D, X, dt, out);
  if (rc == 0)
    for (int64_t i = 0; i < M * D; ++i) out[i] = rnd(out[i] + residual[i], dt);
  free(xn);
  return rc;
}

/* ---------------------------------------------------------------------------------------------
 * LocalAttentionBlock.forward, modules.py:399-493, with its helpers: _apply_rope (modules.py:58-86),
 * _compute_forward_pass_mask / _compute_causal_mask (89-140), _compute_cache_mask (143-163),
 * _attention_cache_from_prompt (238-258), _update_attention_cache (166-196).
 *
 * Multi-query attention: N query heads of dimension Hd = D / N, ONE key/value head.  Rotary
 * embedding on the first half of every head (pairs (i, i + Hd/4) of that half, wavelength 10000),
 * positions = segment_pos.  Prefill (no cache): key s is visible to query t iff s <= t,
 * t <= s + W and both belong to the same document (documents start where segment_pos == 0), t and s
 * being indices in the sequence.  Decode (cache of W slots, T == 1): the cache slot j holds the
 * token of absolute position j + k W (if that is < num_tokens) or j + (k - 1) W, k = num_tokens / W;
 * a slot is visible iff its position is >= 0 and >= num_tokens - W; the new token always is.
 * Roundings in bfloat16 mode: projections (one rounding each), sin / cos cast to bfloat16, every
 * product and sum of the rotation, logits (rounded contraction, then the exact scaling by
 * Hd^-1/2 when that is a power of two, rounded otherwise), softmax in float32 over the masked
 * logits (masked = -2.3819763e38), probabilities cast to bfloat16, the second contraction rounded,
 * proj_final one rounding.
 * ------------------------------------------------------------------------------------------- */
static void rope_inplace(float* x, const int64_t* pos, int64_t rows, int heads, int hd, int dt) {
  /* x [rows, heads, hd]; pos [rows] */
  const int half = hd / 2, quarter = hd / 4;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int i = 0; i < quarter; ++i) {
      const float exponent = 2.0f * (float)i / (float)half;
      const float timescale = powf(10000.0f, exponent);
      const float inv = 1.0f / timescale;
      const float ang = (float)pos[r] * inv;
      const float sn = rnd(sinf(ang), dt), cs = rnd(cosf(ang), dt);
      for (int n = 0; n < heads; ++n) {
        float* h = x + (r * heads + n) * hd;
        const float a = h[i], b = h[i + quarter];
        h[i] = rnd(rnd(a * cs, dt) - rnd(b * sn, dt), dt);
        h[i + quarter] = rnd(rnd(b * cs, dt) + rnd(a * sn, dt), dt);
      }
    }
  }
}

RGO_API void rgo_rope(float* x, const int64_t* pos, int64_t rows, int heads, int hd, int dt) {
  rope_inplace(x, pos, rows, heads, hd, dt);
}

/* q [B,T,N,Hd] (rotated), k / v [B,S,Hd], visible(b,t,s) given as a byte mask [B,T,S]:
 * encoded [B,T,N*Hd] */
static void attention_core(const float* q, const float* k, const float* v, const unsigned char* vis,
                           int B, int T, int S, int N, int Hd, int dt, float* enc) {
  const float scale = 1.0f / sqrtf((float)Hd);
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b) {
    for (int t = 0; t < T; ++t) {
      float* lg = (float*)malloc(sizeof(float) * (size_t)S);
      for (int n = 0; n < N; ++n) {
        const float* qr = q + (((int64_t)b * T + t) * N + n) * Hd;
        float mx = -3.0e38f;
        for (int s = 0; s < S; ++s) {
          const float* kr = k + ((int64_t)b * S + s) * Hd;
          float acc = 0.0f;
          for (int d = 0; d < Hd; ++d) acc += qr[d] * kr[d];
          float l = rnd(rnd(acc, dt) * scale, dt);
          if (!vis[((int64_t)b * T + t) * S + s]) l = -2.3819763e38f;
          lg[s] = l;
          if (l > mx) mx = l;
        }
        float sum = 0.0f;
        for (int s = 0; s < S; ++s) { lg[s] = expf(lg[s] - mx); sum += lg[s]; }
        float* o = enc + ((int64_t)b * T + t) * N * Hd + (int64_t)n * Hd;
        for (int d = 0; d < Hd; ++d) o[d] = 0.0f;
        for (int s = 0; s < S; ++s) {
          const float p = rnd(lg[s] / sum, dt);
          if (p == 0.0f) continue;
          const float* vr = v + ((int64_t)b * S + s) * Hd;
          for (int d = 0; d < Hd; ++d) o[d] += p * vr[d];
        }
        for (int d = 0; d < Hd; ++d) o[d] = rnd(o[d], dt);
      }
      free(lg);
    }
  }
}

/* Prefill (cache_k == NULL) or one decode step (cache given, T == 1).
 * x [B,T,D]; wq [D,D], wk / wv [Hd,D], wf [D,D], bf [D] (nn.Linear layouts);
 * cache_k / cache_v [B,W,Hd], cache_n [B] (int64);  out [B,T,D];
 * new_k / new_v [B,W,Hd], new_n [B] (may be NULL: return_cache = False). */
RGO_API int rgo_attention_block(const float* x, const int64_t* segment_pos, const float* wq,
                                const float* wk, const float* wv, const float* wf, const float* bf,
                                const float* cache_k, const float* cache_v, const int64_t* cache_n,
                                int B, int T, int D, int N, int W, int dt, float* out, float* new_k,
                                float* new_v, int64_t* new_n) {
  const int Hd = D / N;
  const int64_t M = (int64_t)B * T;
  if (cache_k != NULL && T != 1) return -2;
  float* q = (float*)malloc(sizeof(float) * (size_t)(M * D));
  float* k = (float*)malloc(sizeof(float) * (size_t)(M * Hd));
  float* v = (float*)malloc(sizeof(float) * (size_t)(M * Hd));
  float* enc = (float*)malloc(sizeof(float) * (size_t)(M * D));
  if (!q || !k || !v || !enc) { free(q); free(k); free(v); free(enc); return -1; }
  rgo_linear(x, wq, NULL, M, D, D, dt, q);
  rgo_linear(x, wk, NULL, M, D, Hd, dt, k);
  rgo_linear(x, wv, NULL, M, D, Hd, dt, v);
  rope_inplace(q, segment_pos, M, N, Hd, dt);
  rope_inplace(k, segment_pos, M, 1, Hd, dt);
  if (cache_k == NULL) {
    unsigned char* vis = (unsigned char*)malloc((size_t)B * T * T);
    for (int b = 0; b < B; ++b) {
      int* seg = (int*)malloc(sizeof(int) * (size_t)T);
      int c = 0;
      for (int t = 0; t < T; ++t) { if (segment_pos[(int64_t)b * T + t] == 0) ++c; seg[t] = c; }
      for (int t = 0; t < T; ++t)
        for (int s = 0; s < T; ++s)
          vis[((int64_t)b * T + t) * T + s] = (unsigned char)(s <= t && t <= s + W && seg[s] == seg[t]);
      free(seg);
    }
    attention_core(q, k, v, vis, B, T, T, N, Hd, dt, enc);
    free(vis);
    if (new_k != NULL) {
      /* the last w = min(W, T) keys / values, rolled by num_tokens mod W, right padded with zeros */
      const int w = W < T ? W : T;
      for (int b = 0; b < B; ++b) {
        const int64_t nt = segment_pos[(int64_t)b * T + T - 1] + 1;
        new_n[b] = nt;
        for (int64_t i = 0; i < (int64_t)W * Hd; ++i) {
          new_k[(int64_t)b * W * Hd + i] = 0.0f;
          new_v[(int64_t)b * W * Hd + i] = 0.0f;
        }
        const int64_t shift = ((nt % W) + W) % W;
        for (int j = 0; j < w; ++j) {
          /* rolled[j] = tail[(j - shift) mod w] */
          const int64_t src = (((int64_t)j - shift) % w + w) % w;
          const int64_t row = (int64_t)b * T + (T - w) + src;
          for (int d = 0; d < Hd; ++d) {
            new_k[((int64_t)b * W + j) * Hd + d] = k[row * Hd + d];
            new_v[((int64_t)b * W + j) * Hd + d] = v[row * Hd + d];
          }
        }
      }
    }
  } else {
    const int S = W + 1;
    float* kk = (float*)malloc(sizeof(float) * (size_t)B * S * Hd);
    float* vv = (float*)malloc(sizeof(float) * (size_t)B * S * Hd);
    unsigned char* vis = (unsigned char*)malloc((size_t)B * S);
    for (int b = 0; b < B; ++b) {
      const int64_t nt = cache_n[b];
      const int64_t kq = nt / W;
      for (int j = 0; j < W; ++j) {
        const int64_t now = j + kq * W, prev = j + (kq - 1) * W;
        const int64_t kp = now < nt ? now : prev;
        vis[(int64_t)b * S + j] = (unsigned char)(kp >= 0 && nt >= kp && nt <= kp + W);
        for (int d = 0; d < Hd; ++d) {
          kk[((int64_t)b * S + j) * Hd + d] = cache_k[((int64_t)b * W + j) * Hd + d];
          vv[((int64_t)b * S + j) * Hd + d] = cache_v[((int64_t)b * W + j) * Hd + d];
        }
      }
      vis[(int64_t)b * S + W] = 1;
      for (int d = 0; d < Hd; ++d) {
        kk[((int64_t)b * S + W) * Hd + d] = k[(int64_t)b * Hd + d];
        vv[((int64_t)b * S + W) * Hd + d] = v[(int64_t)b * Hd + d];
      }
    }
    attention_core(q, kk, vv, vis, B, 1, S, N, Hd, dt, enc);
    if (new_k != NULL) {
      for (int b = 0; b < B; ++b) {
        const int64_t nt = cache_n[b];
        for (int64_t i = 0; i < (int64_t)W * Hd; ++i) {
          new_k[(int64_t)b * W * Hd + i] = cache_k[(int64_t)b * W * Hd + i];
          new_v[(int64_t)b * W * Hd + i] = cache_v[(int64_t)b * W * Hd + i];
        }
        const int64_t slot = nt % W;
        for (int d = 0; d < Hd; ++d) {
          new_k[((int64_t)b * W + slot) * Hd + d] = k[(int64_t)b * Hd + d];
          new_v[((int64_t)b * W + slot) * Hd + d] = v[(int64_t)b * Hd + d];
        }
        new_n[b] = nt + 1;
      }
    }
    free(kk); free(vv); free(vis);
  }
  rgo_linear(enc, wf, bf, M, D, D, dt, out);
  free(q); free(k); free(v); free(enc);
  return 0;
}

/* ---------------------------------------------------------------------------------------------
 * Labelled restatement of the JAX path's lru_linear_scan (recurrentgemma/jax/scan.py:74-120):
 * h_t = a_t * h_{t-1} + x_t in the accumulation dtype, y_t cast to the dtype of x; `a` is used
 * as given (the caller has already applied the reset mask, jax/layers.py:447-463).
 * ------------------------------------------------------------------------------------------- */
RGO_API void rgo_jax_linear_scan(const float* x, const float* a, const float* h0, int B, int T,
                                 int E, int dt, float* y, float* h_last) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int bi = 0; bi < B; ++bi) {
    for (int e0 = 0; e0 < E; e0 += 64) {
      const int e1 = e0 + 64 < E ? e0 + 64 : E;
      float h[64];
      for (int e = e0; e < e1; ++e) h[e - e0] = h0 ? h0[(int64_t)bi * E + e] : 0.0f;
      for (int t = 0; t < T; ++t) {
        const int64_t row = ((int64_t)bi * T + t) * E;
        for (int e = e0; e < e1; ++e) {
          h[e - e0] = a[row + e] * h[e - e0] + x[row + e];
          y[row + e] = rnd(h[e - e0], dt);
        }
      }
      if (h_last)
        for (int e = e0; e < e1; ++e) h_last[(int64_t)bi * E + e] = h[e - e0];
    }
  }
}
