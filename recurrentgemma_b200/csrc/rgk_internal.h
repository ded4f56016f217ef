// Launchers implemented by the .cu files of librgk; called only from api.cu, which validates
// arguments first.  Each returns the cudaError_t of its last launch.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <mutex>

namespace rgk {

// One-time set-up per device.  cudaFuncSetAttribute applies to the function on the CURRENT device
// only, so a launcher that needs more than the default dynamic shared memory runs its set-up the
// first time it sees each device (a process may drive several), under a lock, and caches that
// device's SM count.  A failed set-up is retried by the next call.
class PerDeviceOnce {
 public:
  template <typename F>
  cudaError_t run(F&& setup, int* num_sms = nullptr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu_);
    if (sms_[dev] == 0) {
      int n = 0;
      if ((e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
      if ((e = setup()) != cudaSuccess) return e;
      sms_[dev] = n;
    }
    if (num_sms != nullptr) *num_sms = sms_[dev];
    return cudaSuccess;
  }

 private:
  static constexpr int kMaxDevices = 64;
  std::mutex mu_;
  int sms_[kMaxDevices] = {};
};

// How the fused RG-LRU kernel evaluates the two sigmoids of the gates and the gelu of the join.
//   kMathExact  sigmoids as 1 / (1 + 2^(-z log2 e)) in float32 with one reciprocal for the four
//               denominators of a token pair (both gates), gelu as z / (1 + 2^w) with one reciprocal
//               per token pair; every rounding of the reference, so that the outputs agree with
//               the reference's bfloat16 arithmetic on all but a fraction of a percent of the elements.
//   kMathFast   the input gate as 0.5 + 0.5 tanh(z / 2) and the gelu as 0.5 z (1 + tanh u) in
//               packed bfloat16 (tanh.approx.bf16x2): 5.5 instead of 6 special-function operations
//               and about 15 fewer instructions per element; a third to a half of the outputs then
//               differ from the reference's by one bfloat16 step.  The recurrence gate keeps the
//               exact form: where a = exp(log_a) sits near 1 a one-step change of that gate flips
//               the rounding of a, and the state of such a slow channel drifts from the reference's.
enum { kMathExact = 0, kMathFast = 1 };

// conv1d.cu
cudaError_t launch_conv1d_prefill(const void* x, const void* pos, int pos64, const void* w,
                                  const void* b, int64_t B, int64_t T, int64_t E, int dtype,
                                  void* out, void* cache_out, cudaStream_t s);
// the cache a prefill returns, alone (the fused RG-LRU kernel computes the convolution itself)
cudaError_t launch_conv1d_cache(const void* x, const void* pos, int pos64, int64_t B, int64_t T,
                                int64_t E, int dtype, void* cache_out, cudaStream_t s);
cudaError_t launch_conv1d_decode(const void* x, const void* cache_in, const void* w, const void* b,
                                 int64_t B, int64_t E, int dtype, void* out, void* cache_out,
                                 cudaStream_t s);

// blockdiag_simt.cu
cudaError_t launch_blockdiag_linear_simt(const void* x, const void* w, const void* b, int64_t M,
                                         int H, int bw, int dtype, void* out, cudaStream_t s);
// Gate projections + gate arithmetic: writes a (reset-masked) and the normalised input.
cudaError_t launch_gates_simt(const void* c, const void* pos, int pos64, const void* a_param,
                              const void* wx, const void* bx, const void* wa, const void* ba,
                              int64_t M, int H, int bw, int dtype, void* a_out, void* xn_out,
                              cudaStream_t s);

// gates_tc.cu: the same as launch_gates_simt on tcgen05 tensor cores (bfloat16, head width 256).
// packed_w: gates_tc_packed_bytes(H) bytes of scratch for the K-major copy of the weights.
bool gates_tc_supported(int dtype, int bw, int64_t M);
size_t gates_tc_packed_bytes(int H);
cudaError_t launch_gates_tc(const void* c, const void* pos, int pos64, const void* a_param,
                            const void* wx, const void* bx, const void* wa, const void* ba,
                            int64_t M, int H, void* packed_w, int packed_ready, void* a_out,
                            void* xn_out, void* ws_header, cudaStream_t s);

// gates_tf32.cu: the same for float32 and head width 256, as three TF32 products per float32
// product (hi/lo split of both operands, float32 accumulation in tensor memory).  packed_w:
// gates_tf32_packed_bytes(H) bytes of scratch for the split K-major copies of the weights.
bool gates_tf32_supported(int dtype, int bw, int64_t M);
size_t gates_tf32_packed_bytes(int H);
cudaError_t launch_pack_gate_weights_tf32(const void* wx, const void* wa, int H, void* packed_w,
                                          cudaStream_t s);
cudaError_t launch_gates_tf32(const void* c, const void* pos, int pos64, const void* a_param,
                              const void* wx, const void* bx, const void* wa, const void* ba,
                              int64_t M, int H, void* packed_w, bool packed_valid, void* a_out, void* xn_out,
                              void* ws_header, cudaStream_t s);

// Packs the gate weights only (the first step of launch_gates_tc), for callers that keep the
// packed copy across calls; launch_gates_tc with packed_ready != 0 then skips its own packing.
cudaError_t launch_pack_gate_weights(const void* wx, const void* wa, int H, void* packed_w,
                                     cudaStream_t s);

// decode_tc.cu: one decode step of the whole sub-path (conv step, gates on tcgen05, state update,
// join) in a single kernel; bfloat16, head width 256.  packed_w as produced by
// launch_pack_gate_weights.  cache_out must not alias cache_in.
cudaError_t launch_path_decode_tc(const void* xb, const void* yb, const void* pos, int pos64,
                                  const void* conv_w, const void* conv_b, const void* a_param,
                                  const void* bx, const void* ba, const void* packed_w,
                                  const float* h_in, const void* cache_in, int64_t B, int H,
                                  void* out, float* h_out, void* cache_out, void* ws_header,
                                  cudaStream_t s, int math);

// rglru_chan_tc.cu: gate projections + gate arithmetic + scan (+ join) in one kernel with
// channel-major accumulators (TMEM lane = channel), so that gate arithmetic, recurrence and join
// run in registers in time order; bfloat16, head width 256, any T.  math: one of the kMath*
// variants of tc_common.cuh (how the sigmoids and the gelu are evaluated).
// ws: rglru_chan_workspace_bytes(B, T, E) bytes whose first word is the caller's status word.
bool rglru_chan_supported(int dtype, int bw, int64_t B, int64_t T);
size_t rglru_chan_workspace_bytes(int64_t B, int64_t T, int64_t E);
cudaError_t launch_rglru_chan(const void* c, const void* pos, int pos64, const void* a_param,
                              const void* bx, const void* ba, const void* packed_w, const float* h0,
                              const void* yb, int y_activated, int64_t B, int64_t T, int H,
                              void* out, float* h_last, void* ws, int math, cudaStream_t s,
                              const void* conv_w = nullptr, const void* conv_b = nullptr);

// gemm_tc.cu: out [M,N] = x [M,K] W[N,K]^T + bias (bfloat16, float32 accumulation) on tcgen05;
// gelu == 1 applies gelu_tanh to the rounded result; gelu == 2 is the GeGLU epilogue of the MLP
// block (W and bias packed by launch_pack_mlp_up, N = 2 X, out [M, X]); residual != null adds a
// [M,N] tensor to the rounded result and rounds again (not together with gelu).  cap != 0 (no bias,
// gelu or residual) is the logits soft cap: tanh(acc / cap) * cap with every rounding of the
// reference.  status: optional device int raised on a bounded-wait timeout.
// gemm_small_tc.cu: the same projection for M <= 256 rows, weights split over all SMs (the K
// slices of a feature tile are a thread-block cluster and add up in distributed shared memory).
// act 0: bias; 1: gelu_tanh of the rounded result; 2: GeGLU over the packed up-projection of the
// MLP (w as pack_mlp_up_kernel writes it, N = 2 X rows, out [M, X]).  w2 != nullptr: a second
// projection of the same x (N2 features, own bias and output) in the same launch; N a multiple of
// 128 then.
bool dense_small_supported(int dtype, int64_t M, int64_t K, int64_t N);
cudaError_t launch_dense_small(const void* x, const void* w, const void* bias, const void* w2,
                               const void* bias2, const void* residual, int64_t M, int K, int N,
                               int N2, int act, void* out, void* out2, int* status, cudaStream_t s);
bool dense_tc_supported(int dtype, int64_t M, int64_t K, int64_t N);
cudaError_t launch_dense_tc(const void* x, const void* w, const void* bias, const void* residual,
                            int64_t M, int K, int N, int gelu, void* out, int* status,
                            cudaStream_t s, float cap = 0.0f);

// attention_decode.cu: one new token per sequence against the ring cache keys / values [B,W,256]
// (num_tokens [B] int32 tokens seen so far): q [B,N,256] and k_new [B,256] rotated, v_new [B,256]
// -> out [B,N*256]; update != 0 then stores k_new / v_new in ring slot num_tokens % W and adds one
// to num_tokens.  ws: attention_decode_workspace_bytes.
bool attention_decode_supported(int hd, int N, int W);
size_t attention_decode_workspace_bytes(int64_t B, int N, int W);
cudaError_t launch_attention_decode(const void* q, const void* k_new, const void* v_new, void* keys,
                                    void* values, int* num_tokens, int64_t B, int N, int W,
                                    int dtype, int update, void* out, void* ws, cudaStream_t s);

// embed.cu: rows of the embedding table scaled by a constant (Embedder.encode), and the index of
// the first maximum of every row of a [M, V] matrix (greedy sampling).
cudaError_t launch_embed(const void* tokens, int tokens64, const void* table, int64_t M, int64_t V,
                         int64_t D, float scale, int dtype, void* out, cudaStream_t s);
cudaError_t launch_argmax(const void* x, int64_t M, int64_t V, int dtype, int* out, cudaStream_t s);
// up [2,M,X], bias [2,X] -> out [M,X] = gelu_tanh(up[0] + bias[0]) * (up[1] + bias[1]), four roundings.
cudaError_t launch_geglu_bias(const void* up, const void* bias, int64_t M, int64_t X, int dtype,
                              void* out, cudaStream_t s);

// ffw_up.w [2, D, X], ffw_up.b [2, X] -> packed_w [2X, D], packed_b [2X] (gemm_tc.cu, mode 3).
cudaError_t launch_pack_mlp_up(const void* w, const void* b, int D, int X, void* packed_w,
                               void* packed_b, cudaStream_t s);

// attention.cu: rotary embedding in place (x [rows, heads, hd], the first half of each head), and
// the local multi-query attention of the attention blocks in prefill form: q [B,T,N,256] and
// k [B,T,256] rotated, v [B,T,256], bfloat16 -> out [B,T,N*256].  ws: attention_workspace_bytes.
cudaError_t launch_rope(void* x, const void* pos, int pos64, int64_t rows, int heads, int hd,
                        int dtype, cudaStream_t s);
bool attention_supported(int dtype, int hd, int64_t B, int64_t T, int N);
size_t attention_workspace_bytes(int64_t B, int64_t T);
cudaError_t launch_attention_prefill(const void* q, const void* k, const void* v, const void* pos,
                                     int pos64, int64_t B, int64_t T, int N, int window, void* out,
                                     void* ws, cudaStream_t s);

// rmsnorm.cu: out [M,D] = x * rsqrt(mean(x^2) + eps) * (scale + 1) with the reference's roundings
// (torch/layers.py:65-73); one warp per row held in registers.
bool rmsnorm_supported(int dtype, int64_t D);
cudaError_t launch_rmsnorm(const void* x, const void* scale, int64_t M, int64_t D, float eps,
                           int dtype, void* out, cudaStream_t s, const void* addend = nullptr,
                           void* sum_out = nullptr);

// scan.cu
size_t scan_workspace_bytes(int64_t B, int64_t T, int64_t E, int dtype);
// y_mul (optional): the join y * gelu_tanh(y_mul), or y * y_mul when y_activated != 0 (the factor
// was already passed through gelu by whoever produced it).  skip_time_tiles / spin_limit: only for
// the wait-expiry self-test (rgk_selftest_wait_expiry); 0 = the whole problem, the default limit.
cudaError_t launch_scan(const void* x, const void* a, const uint8_t* reset, const void* pos,
                        int pos64, const float* h0, const void* y_mul, int y_activated, int64_t B,
                        int64_t T, int64_t E, int dtype, void* y, float* h_last, void* ws,
                        cudaStream_t s, int skip_time_tiles = 0, unsigned spin_limit = 0);

// The scan's built-in scratch (a __device__ array inside scan.cu): its size, and its address on the
// current device (looked up with cudaGetSymbolAddress on first use per device).
size_t scan_static_scratch_bytes();
cudaError_t scan_static_scratch(void** ptr_out);

// decode.cu
// One recurrence step from precomputed a / normalised x: h_out = a h_in + xn (float32, unrounded),
// out = round(h_out) [* gelu_tanh(yb)].
cudaError_t launch_decode_update(const void* a, const void* xn, const float* h_in, const void* yb,
                                 int64_t B, int64_t E, int dtype, void* out, float* h_out,
                                 cudaStream_t s);

}  // namespace rgk
