/*
 * rgk.h - C ABI of librgk.so: the RG-LRU + Conv1D path of recurrentgemma's torch implementation
 * as hand-written CUDA for sm_100a (NVIDIA B200).
 *
 * The reference is pure Python and has no FFI; the interface each entry point replaces is the
 * Python method cited beside it (paths inside the recurrentgemma checkout).  All pointers are
 * DEVICE pointers unless stated otherwise; tensors are dense, row-major and contiguous; nothing is
 * allocated, freed or retained by the library (scratch comes from the caller, see
 * rgk_workspace_bytes; the one exception is rgk_linear_scan_static, which runs on an array built
 * into the library's device image).  Every call only enqueues work on `stream` (a cudaStream_t) and returns
 * 0 or a negative rgk_status; it never synchronises, throws or exits.  There is no CPU path: on a
 * device that is not compute capability 10.x every call returns RGK_EARCH.
 *
 * dtype: activations and parameters are either all float32 or all bfloat16 (RGK_F32 / RGK_BF16).
 * In RGK_BF16 the kernels round after every tensor-level operation of the reference, as torch
 * does for bfloat16 tensors.  The recurrence state is float32 in both (torch/layers.py:146, 376).
 * segment_pos is int32 or int64 (RGK_I32 / RGK_I64); a value of 0 marks the first token of a
 * document (torch/layers.py:335), negative values (left padding, torch/sampler.py:235-238) are
 * ordinary non-zero positions.
 */
#ifndef RGK_H_
#define RGK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RGK_ABI_VERSION 8

#if defined(__GNUC__)
#define RGK_API __attribute__((visibility("default")))
#else
#define RGK_API
#endif

typedef enum rgk_status {
  RGK_OK = 0,
  RGK_EINVAL = -1,     /* null pointer, negative size, unknown enum */
  RGK_ESHAPE = -2,     /* shape the kernels do not cover (message says which) */
  RGK_EALIGN = -3,     /* pointer not 16-byte aligned */
  RGK_EARCH = -4,      /* current device is not sm_100 */
  RGK_ECUDA = -5,      /* a CUDA runtime call failed (message holds cudaGetErrorString) */
  RGK_EWORKSPACE = -6, /* workspace missing or too small */
  RGK_ETIMEOUT = -7,   /* a bounded device-side wait expired (reported by rgk_workspace_status) */
  RGK_EBOUNDS = -8     /* only from a library built with -DRGK_CHECKS: a computed index fell outside
                          its array; the access was skipped (reported by rgk_workspace_status) */
} rgk_status;

enum { RGK_F32 = 0, RGK_BF16 = 1 };
enum { RGK_I32 = 0, RGK_I64 = 1 };

/* Which kernels a composed call may use for the block-diagonal gate projections. */
enum {
  RGK_GATES_AUTO = 0,    /* the fastest kernel that covers the shape (see below) */
  RGK_GATES_SIMT = 1,    /* CUDA-core gate kernel, then the scan kernel (any head width that is a
                            multiple of 16; float32 or bfloat16) */
  RGK_GATES_TCGEN05 = 2, /* tensor-core gate kernel, then the scan kernel (head width 256: bfloat16,
                            or float32 as three TF32 products per float32 product); RGK_ESHAPE if
                            the shape is not covered */
  RGK_GATES_FUSED = 3,   /* gates, gate arithmetic and scan in one tensor-core kernel (bfloat16,
                            head width 256, any T); RGK_ESHAPE otherwise.  The input gate and the
                            gelu of the join are evaluated with packed bfloat16 tanh approximations:
                            within the path's tolerance of the reference (2e-2 of the largest
                            output), a third to a half of the outputs differ by one bfloat16 step */
  RGK_GATES_FUSED_EXACT = 4 /* the same kernel with every rounding of the reference (sigmoids and
                            gelu in float32 before their rounding): outputs agree with the
                            reference's bfloat16 arithmetic on all but a fraction of a percent of
                            the elements; about 10 % slower */
};

RGK_API int rgk_abi_version(void);

/* Thread-local text of the last failure on the calling host thread ("" if none). */
RGK_API const char* rgk_last_error(void);

/* RGK_OK if the current CUDA device can run this library, else RGK_EARCH / RGK_ECUDA. */
RGK_API int rgk_device_check(void);

/* ------------------------------------------------------------------------------------------------
 * Conv1D.forward, prefill form (cache is None)                    torch/layers.py:447-529
 *   x [B,T,E], segment_pos [B,T], w [W,E], b [E]  ->  out [B,T,E], cache_out [B,W-1,E] or NULL
 * Causal depthwise convolution whose taps do not cross a document start; cache_out receives the
 * last W-1 input rows as the reference leaves them (masked by later document starts, zero where
 * T < W-1).  W must be 4.  x is not modified.
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_conv1d_prefill(const void* x, const void* segment_pos, int pos_dtype, const void* w,
                       const void* b, int64_t B, int64_t T, int64_t E, int W, int dtype, void* out,
                       void* cache_out, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Conv1D.forward, decode form (cache given, T == 1)               torch/layers.py:469-474, 531-550
 *   x [B,E], cache_in [B,W-1,E]  ->  out [B,E], cache_out [B,W-1,E] (may alias cache_in) or NULL
 * No document masking in this form.  W must be 4.
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_conv1d_decode(const void* x, const void* cache_in, const void* w, const void* b, int64_t B,
                      int64_t E, int W, int dtype, void* out, void* cache_out, void* stream);

/* ------------------------------------------------------------------------------------------------
 * BlockDiagonalLinear.forward                                      torch/layers.py:127-137
 *   x [M, H*bw], w [H, bw(in), bw(out)], b [H, bw]  ->  out [M, H*bw]
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_blockdiag_linear(const void* x, const void* w, const void* b, int64_t M, int H, int bw,
                         int dtype, void* out, void* stream);

/* ------------------------------------------------------------------------------------------------
 * rnn_scan                                                         torch/layers.py:140-191
 *   x, a [B,T,E] (dtype), reset [B,T] uint8 (non-zero = reset), h0 [B,E] float32 or NULL
 *   ->  y [B,T,E] (dtype), h_last [B,E] float32 or NULL
 * h_t = (a_t * !reset_t) * h_{t-1} + x_t in float32; with T == 1 and h0 == NULL the output is x
 * (torch/layers.py:172-173).  y_mul (optional, [B,T,E]) fuses RecurrentBlock's join
 * (torch/modules.py:627-628, 646): y <- y * gelu_tanh(y_mul).
 * workspace: rgk_workspace_bytes(B, T, E, dtype) bytes, 256-byte aligned; reused freely between
 * calls that do not overlap on the device.
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_linear_scan(const void* x, const void* a, const uint8_t* reset, const float* h0,
                    const void* y_mul, int64_t B, int64_t T, int64_t E, int dtype, void* y,
                    float* h_last, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * rgk_linear_scan for callers that cannot allocate device memory.  (No counterpart in the
 * reference: it exists for hosts such as a serving runtime that plans all device buffers up front
 * and forbids allocation on its request path, or a process whose own arena already owns the whole
 * device, so that a cudaMalloc made on the library's behalf would fail.)
 *
 * Same computation and arguments as rgk_linear_scan, minus the workspace: the scratch is an 8 MiB
 * array built into the library's device image (held by every GPU that loads the library until the
 * process exits).  Problems whose scan scratch exceeds 8 MiB - about 10,800 tiles of 128 x 64
 * elements in bfloat16 (64 x 64 in float32); B8 T4096 E2560 bfloat16 fits - are rejected with
 * RGK_ESHAPE.  The call allocates nothing: no cudaMalloc / cudaFree, only launches, memsets and
 * one 4-byte device-to-device copy.
 *
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call outside any stream capture.  All calls on a device share the one array:
 * two calls that overlap on the GPU (different streams, no ordering between them) race and give
 * wrong results; calls on one stream, or otherwise ordered, are fine, and no state has to be
 * cleared by the caller between them.
 *
 * status_out (optional, device pointer to one int): receives 0, or RGK_ETIMEOUT if a bounded
 * device-side wait expired, once the call's work on `stream` has finished.
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_linear_scan_static(const void* x, const void* a, const uint8_t* reset,
                                   const float* h0, const void* y_mul, int64_t B, int64_t T,
                                   int64_t E, int dtype, void* y, float* h_last, int* status_out,
                                   void* stream);

/* ------------------------------------------------------------------------------------------------
 * Parameters of one recurrent block's RG-LRU + Conv1D, as the reference state_dict holds them
 * (torch/layers.py:105-112, 262-278, 409-412).
 * ---------------------------------------------------------------------------------------------- */
typedef struct rgk_params {
  const void* conv_w;    /* conv_1d.w            [W, E]            */
  const void* conv_b;    /* conv_1d.b            [E]               */
  const void* a_param;   /* rg_lru.a_param       [E]               */
  const void* gate_x_w;  /* rg_lru.input_gate.w  [H, E/H, E/H] (in, out) */
  const void* gate_x_b;  /* rg_lru.input_gate.b  [H, E/H]          */
  const void* gate_a_w;  /* rg_lru.a_gate.w      [H, E/H, E/H]     */
  const void* gate_a_b;  /* rg_lru.a_gate.b      [H, E/H]          */
  const void* gates_packed; /* optional: output of rgk_pack_gate_weights for these gate weights;
                               NULL makes the tensor-core kernels pack into the workspace per call */
} rgk_params;

/* ------------------------------------------------------------------------------------------------
 * K-major copy of the two gate weights for the tcgen05 kernels (head width 256 only; for float32
 * the hi and lo halves of the 3xTF32 split): rgk_gate_pack_bytes_for(H, dtype) bytes
 * (rgk_gate_pack_bytes(H) = the bfloat16 size), written once per weight update and passed as
 * rgk_params.gates_packed afterwards, with parameters of the same dtype (saves a repack per call;
 * matters for decode steps and short sequences).
 * No reference counterpart: the reference keeps only the [H, in, out] layout
 * (torch/layers.py:105-112).
 * ---------------------------------------------------------------------------------------------- */
RGK_API size_t rgk_gate_pack_bytes(int H);
RGK_API size_t rgk_gate_pack_bytes_for(int H, int dtype);
RGK_API int rgk_pack_gate_weights(const rgk_params* p, int H, int bw, int dtype, void* packed_out,
                                  void* stream);

/* ------------------------------------------------------------------------------------------------
 * RGLRU.forward                                                    torch/layers.py:313-365
 *   x [B,T,E], segment_pos [B,T], h0 [B,E] float32 or NULL
 *   ->  y [B,T,E], h_last [B,E] float32 or NULL
 * Uses a_param and the two gate projections of `p` (conv_w / conv_b are ignored).  Any T >= 1;
 * T == 1 follows the sampling branch of rnn_scan (new state = unrounded float32).
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_rglru_forward(const void* x, const void* segment_pos, int pos_dtype, const rgk_params* p,
                      const float* h0, int64_t B, int64_t T, int64_t E, int H, int dtype,
                      int gates_impl, void* y, float* h_last, void* workspace,
                      size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * The RG-LRU + Conv1D sub-path of RecurrentBlock.forward           torch/modules.py:631-646
 *   prefill:  out = RGLRU(Conv1D(xb)) * gelu_tanh(yb)     (yb NULL: no join, out = RGLRU(Conv1D(xb)))
 *   xb, yb [B,T,E] = linear_x(x), linear_y(x);  h0 [B,E] float32 or NULL
 *   ->  out [B,T,E], h_last [B,E] float32 or NULL, conv_cache_out [B,W-1,E] or NULL
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_recurrent_path_prefill(const void* xb, const void* yb, const void* segment_pos,
                               int pos_dtype, const rgk_params* p, const float* h0, int64_t B,
                               int64_t T, int64_t E, int H, int W, int dtype, int gates_impl,
                               void* out, float* h_last, void* conv_cache_out, void* workspace,
                               size_t workspace_bytes, void* stream);

/* Process-wide switch: with enabled != 0 the bfloat16 / head-width-256 prefill of the sub-path (and
 * of the block entry points built on it) computes the Conv1D inside the RG-LRU kernel - two extra
 * warps per CTA turn the block input into the kernel's conv-output operand, so the conv output
 * never reaches HBM - instead of running rgk_conv1d_prefill's kernel first.  The results are the
 * same bits.  Off by default: measured on a B200 the fused form is the slower one (DRAM traffic
 * falls by a third, but the kernel is bound by instruction issue, not by HBM).  Returns the
 * previous setting. */
RGK_API int rgk_set_conv_fusion(int enabled);

/* ------------------------------------------------------------------------------------------------
 * The same sub-path for one decode step (T == 1 with caches)       torch/modules.py:631-646,
 *   xb, yb [B,E]; conv_cache_in [B,W-1,E]; h_in [B,E] float32     torch/layers.py:170-177, 469-474
 *   ->  out [B,E], h_out [B,E] float32, conv_cache_out [B,W-1,E]
 * h_out may alias h_in and conv_cache_out may alias conv_cache_in (in-place state update: the
 * fused single-kernel step reads and then writes every state element from one and the same
 * thread, so it runs in place as well).
 * segment_pos [B] still selects the reset behaviour of the RG-LRU (a position of 0 drops h_in).
 * gates_impl: RGK_GATES_AUTO / RGK_GATES_FUSED = the single kernel with the packed-tanh input gate
 * and gelu and the table for exp(log_a) (as the prefill kernel's default arithmetic);
 * RGK_GATES_FUSED_EXACT / RGK_GATES_TCGEN05 = the same kernel with every rounding of the reference;
 * RGK_GATES_SIMT = the CUDA-core kernels.
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_recurrent_path_decode(const void* xb, const void* yb, const void* segment_pos,
                              int pos_dtype, const rgk_params* p, const float* h_in,
                              const void* conv_cache_in, int64_t B, int64_t E, int H, int W,
                              int dtype, int gates_impl, void* out, float* h_out,
                              void* conv_cache_out, void* workspace, size_t workspace_bytes,
                              void* stream);

/* ------------------------------------------------------------------------------------------------
 * torch.nn.Linear as the block uses it                              torch/modules.py:531-548
 *   x [M,K], weight [N,K] (out, in), bias [N] or NULL  ->  out [M,N] = x weight^T + bias
 * tcgen05 tensor-core GEMM, bfloat16 only (float32 accumulation, one rounding); K and N multiples
 * of 8.  act: RGK_ACT_NONE, or RGK_ACT_GELU_TANH to apply gelu(approximate="tanh") to the rounded
 * result (torch/modules.py:289-291, 628).  status (optional device int) is raised to RGK_ETIMEOUT if
 * a bounded device-side wait expires.
 * ---------------------------------------------------------------------------------------------- */
enum { RGK_ACT_NONE = 0, RGK_ACT_GELU_TANH = 1, RGK_ACT_GEGLU = 2 /* rgk_dense_linear_small only */ };
RGK_API int rgk_dense_linear(const void* x, const void* weight, const void* bias, int64_t M,
                             int64_t K, int64_t N, int dtype, int act, void* out, int* status,
                             void* stream);

/* ------------------------------------------------------------------------------------------------
 * The same torch.nn.Linear for FEW rows (M <= 256: a decode step, where M is the batch)
 *                                                        torch/modules.py:437-452, 531-548, 626-647
 *   x [M,K], weight [N,K], bias [N] or NULL, residual [M,N] or NULL
 *   ->  out [M,N] = act(x weight^T + bias) (+ residual, rounded once more, when given)
 * The weights are split over all SMs (128 output features x a slice of K per CTA) so that the
 * call streams them once at HBM speed; the K slices of a feature tile form a thread-block cluster
 * and add their float32 partial sums in distributed shared memory in a fixed order (the same bits
 * on every run).  The kernel is launched with programmatic stream serialisation: it may begin
 * (fetching weights) while the kernel before it in the stream drains, and touches nothing else
 * before that kernel has completed.  bfloat16 only, K and N multiples of 8; RGK_ESHAPE otherwise
 * (M > 256 included: rgk_dense_linear covers those).  Roundings as rgk_dense_linear.  status as there.
 * act RGK_ACT_GEGLU: the up-projection of the MLP block (torch/modules.py:749-752): weight and
 *   bias are the packed copy rgk_pack_mlp_up writes (N = 2 X rows, X a multiple of 64), out [M, X]
 *   = gelu_tanh(gate) * value with the roundings of rgk_mlp_block; no residual.
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_dense_linear_small(const void* x, const void* weight, const void* bias,
                                   const void* residual, int64_t M, int64_t K, int64_t N, int dtype,
                                   int act, void* out, int* status, void* stream);
/* Two projections of the same x in one launch (linear_y and linear_x of the recurrent block,
 * torch/modules.py:626-631; proj_k and proj_v of the attention block, torch/modules.py:437-452):
 *   out_a [M,N_a] = x weight_a^T + bias_a,  out_b [M,N_b] = x weight_b^T + bias_b   (biases or NULL)
 * N_a a multiple of 128; otherwise as rgk_dense_linear_small with RGK_ACT_NONE. */
RGK_API int rgk_dense_linear_small_pair(const void* x, const void* weight_a, const void* bias_a,
                                        const void* weight_b, const void* bias_b, int64_t M,
                                        int64_t K, int64_t N_a, int64_t N_b, int dtype, void* out_a,
                                        void* out_b, int* status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * RecurrentBlock.forward, prefill form (cache is None)              torch/modules.py:605-655
 *   x [B,T,D]  ->  out [B,T,D], h_last [B,E] float32 or NULL, conv_cache_out [B,W-1,E] or NULL
 * linear_y (+gelu) and linear_x on tensor cores, the RG-LRU + Conv1D sub-path, linear_out.
 * bfloat16 with head width 256 only (RGK_ESHAPE otherwise: compose the calls above instead).
 * workspace: rgk_block_workspace_bytes(B, T, D, E, dtype) bytes, 256-byte aligned.
 * ---------------------------------------------------------------------------------------------- */
typedef struct rgk_block_params {
  rgk_params path;           /* conv_1d.*, rg_lru.*                         */
  const void* linear_y_w;    /* linear_y.weight   [E, D]                    */
  const void* linear_y_b;    /* linear_y.bias     [E]                       */
  const void* linear_x_w;    /* linear_x.weight   [E, D]                    */
  const void* linear_x_b;    /* linear_x.bias     [E]                       */
  const void* linear_out_w;  /* linear_out.weight [D, E]                    */
  const void* linear_out_b;  /* linear_out.bias   [D]                       */
} rgk_block_params;
RGK_API size_t rgk_block_workspace_bytes(int64_t B, int64_t T, int64_t D, int64_t E, int dtype);
RGK_API int rgk_recurrent_block_prefill(const void* x, const void* segment_pos, int pos_dtype,
                                        const rgk_block_params* p, int64_t B, int64_t T, int64_t D,
                                        int64_t E, int H, int W, int dtype, void* out,
                                        float* h_last, void* conv_cache_out, void* workspace,
                                        size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * RMSNorm.forward (recurrentgemma/torch/layers.py:65-73) over the last dimension of x [M, D]:
 *   out = x * rsqrt(mean(x^2) + eps) * (scale + 1)
 * with one rounding per tensor operation of the reference in bfloat16.  D a multiple of the
 * 16-byte pack (8 bfloat16 / 4 float32) and at most 1024 packs; RGK_ESHAPE otherwise.
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_rmsnorm(const void* x, const void* scale, int64_t M, int64_t D, float eps, int dtype,
                        void* out, void* stream);
/* The same with the residual add in front (recurrentgemma/torch/modules.py:902-904):
 * sum_out [M,D] = a + b (one rounding), out [M,D] = RMSNorm(sum_out). */
RGK_API int rgk_add_rmsnorm(const void* a, const void* b, const void* scale, int64_t M, int64_t D,
                            float eps, int dtype, void* sum_out, void* out, void* stream);

/* ------------------------------------------------------------------------------------------------
 * The temporal half of ResidualBlock.forward for a recurrent block
 * (recurrentgemma/torch/modules.py:897-902), prefill form:
 *   out = RecurrentBlock(RMSNorm(x; norm_scale)) + x
 * RMSNorm runs as its own kernel, the residual is added in the epilogue of linear_out's GEMM.
 * Same coverage and outputs as rgk_recurrent_block_prefill.
 * workspace: rgk_residual_workspace_bytes(B, T, D, E, dtype) bytes, 256-byte aligned.
 * ---------------------------------------------------------------------------------------------- */
RGK_API size_t rgk_residual_workspace_bytes(int64_t B, int64_t T, int64_t D, int64_t E, int dtype);
RGK_API int rgk_residual_block_prefill(const void* x, const void* segment_pos, int pos_dtype,
                                       const rgk_block_params* p, const void* norm_scale, float eps,
                                       int64_t B, int64_t T, int64_t D, int64_t E, int H, int W,
                                       int dtype, void* out, float* h_last, void* conv_cache_out,
                                       void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * MLPBlock.forward (recurrentgemma/torch/modules.py:740-752) and the channel half of
 * ResidualBlock.forward (torch/modules.py:904-908), bfloat16:
 *   mlp(x)   = ffw_down( gelu_tanh(x w_up[0] + b_up[0]) * (x w_up[1] + b_up[1]) )
 *   channel  = mlp(RMSNorm(r; norm_scale)) + r
 * ffw_up runs as ONE tcgen05 GEMM over weights packed gate/value-interleaved and K-major
 * (rgk_pack_mlp_up: w_up [2, D, X] (in, out), b_up [2, X] -> rgk_mlp_pack_bytes(D, X) bytes, once
 * per set of weights) whose epilogue forms gelu(gate) * value, so the [M, 2X] pre-activations never
 * reach HBM; ffw_down is the dense GEMM with the optional residual [M, D] added in its epilogue.
 * D a multiple of 8, X a multiple of 64; RGK_ESHAPE otherwise and for float32.
 * workspace: rgk_mlp_workspace_bytes(M, D, X, dtype) bytes, 256-byte aligned (its first word is the
 * status word of rgk_workspace_status).
 * ---------------------------------------------------------------------------------------------- */
RGK_API size_t rgk_mlp_pack_bytes(int64_t D, int64_t X);
RGK_API int rgk_pack_mlp_up(const void* w_up, const void* b_up, int64_t D, int64_t X, int dtype,
                            void* packed_out, void* stream);
RGK_API size_t rgk_mlp_workspace_bytes(int64_t M, int64_t D, int64_t X, int dtype);
RGK_API int rgk_mlp_block(const void* x, const void* packed_up, const void* down_w,
                          const void* down_b, const void* residual, int64_t M, int64_t D, int64_t X,
                          int dtype, void* out, void* workspace, size_t workspace_bytes,
                          void* stream);
RGK_API int rgk_residual_channel(const void* residual_in, const void* norm_scale, float eps,
                                 const void* packed_up, const void* down_w, const void* down_b,
                                 int64_t M, int64_t D, int64_t X, int dtype, void* out,
                                 void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Pieces of LocalAttentionBlock.forward (recurrentgemma/torch/modules.py:399-493).
 * rgk_rope: _apply_rope (torch/modules.py:58-86) in place on x [rows, heads, head_dim], positions
 *   [rows]: the first half of every head is rotated, float32 or bfloat16.
 * rgk_local_attention_prefill: the attention proper without a cache - logits of rotated queries
 *   q [B,T,N,head_dim] and keys k [B,T,head_dim] (one key/value head), the causal / window / same
 *   document mask of torch/modules.py:89-140, float32 softmax of the bfloat16-rounded logits,
 *   probabilities rounded to bfloat16, product with v [B,T,head_dim] -> out [B,T,N*head_dim].
 *   bfloat16 with head_dim 256; RGK_ESHAPE otherwise.
 * workspace: rgk_attention_workspace_bytes(B, T) bytes, 256-byte aligned (first word: status).
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_rope(void* x, const void* segment_pos, int pos_dtype, int64_t rows, int heads,
                     int head_dim, int dtype, void* stream);
RGK_API size_t rgk_attention_workspace_bytes(int64_t B, int64_t T);
RGK_API int rgk_local_attention_prefill(const void* q, const void* k, const void* v,
                                        const void* segment_pos, int pos_dtype, int64_t B, int64_t T,
                                        int N, int head_dim, int window, int dtype, void* out,
                                        void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * LocalAttentionBlock.forward with a cache: one new token per sequence against the ring buffer
 * (recurrentgemma/torch/modules.py:437-476, mask of torch/modules.py:155-184, ring update of
 * torch/modules.py:187-286).
 *   q [B,N,head_dim] and k_new [B,head_dim] rotated (rgk_rope), v_new [B,head_dim];
 *   keys, values [B,W,head_dim] (the cache's [B,W,1,head_dim]), num_tokens [B] int32
 *   ->  out [B,N*head_dim]: bfloat16-rounded scaled logits over the W ring entries the query sees
 *   (positions num_tokens - W .. num_tokens - 1) and the new key, float32 softmax, probabilities
 *   rounded, product with the values.  update != 0: afterwards k_new / v_new are stored in ring slot
 *   num_tokens % W and num_tokens grows by one, all in place (clone the cache first for the
 *   reference's functional form).  float32 or bfloat16, head_dim 256, N in {1,2,4,8,10};
 *   RGK_ESHAPE otherwise.
 * workspace: rgk_attention_decode_workspace_bytes(B, N, W) bytes, 256-byte aligned.
 * ---------------------------------------------------------------------------------------------- */
RGK_API size_t rgk_attention_decode_workspace_bytes(int64_t B, int N, int window);
RGK_API int rgk_local_attention_decode(const void* q, const void* k_new, const void* v_new,
                                       void* keys, void* values, int* num_tokens, int64_t B, int N,
                                       int head_dim, int window, int dtype, int update, void* out,
                                       void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * The two ends of Griffin.forward around the residual blocks, and greedy sampling.
 * rgk_embed: Embedder.encode (recurrentgemma/torch/modules.py:991-998): out [M,D] =
 *   table[tokens[m], :] * scale (scale = sqrt(D) rounded to bfloat16, or 1), tokens RGK_I32 or
 *   RGK_I64, float32 or bfloat16, D a multiple of a 16-byte pack.  A token outside
 *   [0, V) reads the nearest row (the reference raises).
 * rgk_logits: Embedder.decode followed by the soft cap (torch/modules.py:1001-1003,
 *   torch/griffin.py:180-185): out [M,V] = x [M,D] table[V,D]^T, then tanh(. / cap) * cap when
 *   cap != 0, with the bfloat16 rounding of each of the reference's tensor operations.  tcgen05
 *   GEMM, bfloat16 only, D and V multiples of 8.  status: as for rgk_dense_linear.
 * rgk_argmax: torch.argmax(logits, dim=-1) (torch/sampler.py:131-132): out [M] int32 = index of
 *   the first maximum of every row of x [M,V], float32 or bfloat16.
 * ---------------------------------------------------------------------------------------------- */
RGK_API int rgk_embed(const void* tokens, int token_dtype, const void* table, int64_t M, int64_t V,
                      int64_t D, float scale, int dtype, void* out, void* stream);
RGK_API int rgk_logits(const void* x, const void* table, int64_t M, int64_t D, int64_t V, float cap,
                       int dtype, void* out, int* status, void* stream);
RGK_API int rgk_argmax(const void* x, int64_t M, int64_t V, int dtype, int* out, void* stream);

/* The element-wise part of MLPBlock.forward (recurrentgemma/torch/layers.py:700-703,
 * torch/modules.py:749-751) for callers that contract ffw_up elsewhere (a decode step of a few
 * rows): up [2,M,X] (the two contractions, rounded), bias [2,X]  ->  out [M,X] =
 * gelu_tanh(up[0] + bias[0]) * (up[1] + bias[1]), each of the four tensor operations rounded.
 * float32 or bfloat16; X a multiple of a 16-byte pack. */
RGK_API int rgk_geglu_bias(const void* up, const void* bias, int64_t M, int64_t X, int dtype,
                           void* out, void* stream);

/* Scratch needed by the calls above for a problem of this size (an upper bound over the entry
 * points, so one buffer serves all of them).  Returns 0 on invalid arguments. */
RGK_API size_t rgk_workspace_bytes(int64_t B, int64_t T, int64_t E, int dtype);

/* The first int of a workspace is its status word.  Kernels only ever RAISE it (to RGK_ETIMEOUT,
 * when a bounded device-side wait gave up); no call of this library clears it, so the word tells
 * whether anything went wrong on this workspace since the caller last cleared it.  A new workspace
 * must start with the word at 0 (cudaMemset the first 4 bytes once).
 * rgk_workspace_status synchronises `stream`, copies the word to the host and returns RGK_OK or
 * RGK_ETIMEOUT; a raised word is cleared as it is reported. */
RGK_API int rgk_workspace_status(void* workspace, void* stream);

/* Self-test of the failure path (no counterpart in the reference): runs a small scan in which the
 * records of the first time tile are never published, with the poll limit of the look-back lowered
 * to 200, so that the bounded waits of the next tile run out within microseconds.  The kernel must
 * finish by itself and leave RGK_ETIMEOUT in the status word (rgk_workspace_status then returns
 * it).  Nothing faults, traps or waits without a limit.  workspace: at least 1 MiB, 256-byte
 * aligned; its contents are overwritten. */
RGK_API int rgk_selftest_wait_expiry(void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RGK_H_ */
