// extern "C" surface of librgk (include/rgk.h): argument validation, error text, workspace carving
// and the composition of the kernels into the calls the reference's Python methods map to.
#include <cstdarg>
#include <cstdio>
#include <atomic>
#include <cstring>

#include "../../include/rgk.h"
#include "rgk_common.cuh"
#include "rgk_internal.h"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(RGK_ECUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

int elem_size(int dtype) { return dtype == RGK_BF16 ? 2 : 4; }

// Compute capability of each device, looked up once (immutable afterwards).
int device_ok() {
  static int cached[64];  // 0 unknown, 1 ok, -1 wrong arch
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev >= 0 && dev < 64 && cached[dev] == 1) return RGK_OK;
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
  if (major != 10) {
    return fail(RGK_EARCH, "device %d has compute capability %d.x; librgk is built for sm_100a only",
                dev, major);
  }
  if (dev >= 0 && dev < 64) cached[dev] = 1;
  return RGK_OK;
}

#define RGK_REQUIRE(cond, code, ...) \
  do {                               \
    if (!(cond)) return fail(code, __VA_ARGS__); \
  } while (0)

#define RGK_CHECK_DEVICE()          \
  do {                              \
    int rc_ = device_ok();          \
    if (rc_ != RGK_OK) return rc_;  \
  } while (0)

#define RGK_CUDA(expr, what)                              \
  do {                                                    \
    cudaError_t e_ = (expr);                              \
    if (e_ != cudaSuccess) return cuda_fail(e_, what);    \
  } while (0)

int check_common(int64_t B, int64_t T, int64_t E, int dtype) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(B >= 0 && T >= 0 && E >= 0, RGK_EINVAL, "negative size (B=%lld T=%lld E=%lld)",
              (long long)B, (long long)T, (long long)E);
  const int pack = dtype == RGK_BF16 ? 8 : 4;
  RGK_REQUIRE(E % pack == 0, RGK_ESHAPE, "width %lld is not a multiple of %d (16-byte channel packs)",
              (long long)E, pack);
  RGK_REQUIRE(B <= 65535, RGK_ESHAPE, "batch %lld exceeds 65535", (long long)B);
  RGK_REQUIRE(T <= (1 << 21), RGK_ESHAPE, "sequence length %lld exceeds 2^21", (long long)T);
  RGK_REQUIRE(E <= (1 << 20), RGK_ESHAPE, "width %lld exceeds 2^20", (long long)E);
  return RGK_OK;
}

int check_heads(int64_t E, int H) {
  RGK_REQUIRE(H >= 1 && E % H == 0, RGK_ESHAPE, "width %lld is not divisible by %d heads",
              (long long)E, H);
  RGK_REQUIRE((E / H) % 16 == 0, RGK_ESHAPE, "head width %lld is not a multiple of 16",
              (long long)(E / H));
  return RGK_OK;
}

int check_params(const rgk_params* p, bool need_conv) {
  RGK_REQUIRE(p != nullptr, RGK_EINVAL, "params is NULL");
  RGK_REQUIRE(p->a_param && p->gate_x_w && p->gate_x_b && p->gate_a_w && p->gate_a_b, RGK_EINVAL,
              "a gate parameter pointer is NULL");
  RGK_REQUIRE(!need_conv || (p->conv_w && p->conv_b), RGK_EINVAL, "conv parameter pointer is NULL");
  RGK_REQUIRE(aligned16(p->a_param) && aligned16(p->gate_x_w) && aligned16(p->gate_x_b) &&
                  aligned16(p->gate_a_w) && aligned16(p->gate_a_b) &&
                  (!need_conv || (aligned16(p->conv_w) && aligned16(p->conv_b))),
              RGK_EALIGN, "parameter pointers must be 16-byte aligned");
  return RGK_OK;
}

// Gate projections + gate arithmetic with the kernel `gates_impl` selects.
int run_gates(const void* c, const void* pos, int pos64, const rgk_params* p, int64_t M, int H,
              int bw, int dtype, int gates_impl, void* wpack, void* a, void* xn, void* ws_header,
              cudaStream_t s) {
  const bool tc_ok = rgk::gates_tc_supported(dtype, bw, M);
  const bool tf32_ok = rgk::gates_tf32_supported(dtype, bw, M);
  if (gates_impl == RGK_GATES_TCGEN05 && !tc_ok && !tf32_ok)
    return fail(RGK_ESHAPE, "the tcgen05 gate kernels cover head width 256 only "
                            "(dtype %d, head width %d)", dtype, bw);
  if (tf32_ok && gates_impl != RGK_GATES_SIMT) {
    cudaError_t e = rgk::launch_gates_tf32(c, pos, pos64, p->a_param, p->gate_x_w, p->gate_x_b,
                                           p->gate_a_w, p->gate_a_b, M, H,
                                           p->gates_packed ? const_cast<void*>(p->gates_packed) : wpack,
                                           p->gates_packed != nullptr, a, xn, ws_header, s);
    if (e != cudaSuccess) return cuda_fail(e, "tcgen05 TF32 gates launch");
    return RGK_OK;
  }
  if (tc_ok && gates_impl != RGK_GATES_SIMT) {
    cudaError_t e = rgk::launch_gates_tc(
        c, pos, pos64, p->a_param, p->gate_x_w, p->gate_x_b, p->gate_a_w, p->gate_a_b, M, H,
        p->gates_packed ? const_cast<void*>(p->gates_packed) : wpack, p->gates_packed != nullptr, a,
        xn, ws_header, s);
    if (e != cudaSuccess) return cuda_fail(e, "tcgen05 gates launch");
    return RGK_OK;
  }
  cudaError_t e = rgk::launch_gates_simt(c, pos, pos64, p->a_param, p->gate_x_w, p->gate_x_b,
                                         p->gate_a_w, p->gate_a_b, M, H, bw, dtype, a, xn, s);
  if (e != cudaSuccess) return cuda_fail(e, "gates launch");
  return RGK_OK;
}

// Whether the prefill path convolves inside the fused RG-LRU kernel (rgk_set_conv_fusion).  Off by
// default: on a B200 the two conv warps a CTA can afford cannot keep up with its sixteen epilogue
// warps (the same bits, at about half the speed of the separate conv kernel).
static std::atomic<int> g_conv_fusion{0};
static bool conv_fusion_enabled() { return g_conv_fusion.load(std::memory_order_relaxed) != 0; }

// RG-LRU on a conv output c: fused kernel when asked for / possible, else gates then scan.
// With xb != nullptr the Conv1D is this function's job as well: `c` is then only a buffer for the
// conv output, which the fused kernel does not need (it convolves xb itself, unless out aliases
// xb: the units read each other's input rows) and the other routes fill with conv1d_prefill.
int run_rglru(const void* c, const void* pos, int pos64, const rgk_params* p, const float* h0,
              const void* yb, int y_activated, int64_t B, int64_t T, int64_t E, int H, int dtype,
              int gates_impl, void* wpack, void* a_buf, void* xn_buf, void* scan_ws, void* out,
              float* h_last, cudaStream_t s, const void* xb = nullptr, void* conv_cache_out = nullptr) {
  const int bw = (int)(E / H);
  const bool chan_route = rgk::rglru_chan_supported(dtype, bw, B, T) &&
                          (gates_impl == RGK_GATES_AUTO || gates_impl >= RGK_GATES_FUSED);
  const bool fuse_conv = xb != nullptr && chan_route && out != xb && conv_fusion_enabled();
  if (xb != nullptr) {
    cudaError_t e = fuse_conv
        ? rgk::launch_conv1d_cache(xb, pos, pos64, B, T, E, dtype, conv_cache_out, s)
        : rgk::launch_conv1d_prefill(xb, pos, pos64, p->conv_w, p->conv_b, B, T, E, dtype,
                                     const_cast<void*>(c), conv_cache_out, s);
    if (e != cudaSuccess) return cuda_fail(e, "conv1d launch");
  }
  const bool fused_ok = rgk::rglru_chan_supported(dtype, bw, B, T);
  const bool want_fused = gates_impl >= RGK_GATES_FUSED;
  if (want_fused && !fused_ok)
    return fail(RGK_ESHAPE, "the fused RG-LRU kernel covers bfloat16 and head width 256 "
                            "(dtype %d, head width %d, T %lld)", dtype, bw, (long long)T);
  if (fused_ok && (gates_impl == RGK_GATES_AUTO || want_fused)) {
    const int math = gates_impl == RGK_GATES_FUSED_EXACT ? rgk::kMathExact : rgk::kMathFast;
    const void* packed = p->gates_packed;
    if (packed == nullptr) {
      cudaError_t e = rgk::launch_pack_gate_weights(p->gate_x_w, p->gate_a_w, H, wpack, s);
      if (e != cudaSuccess) return cuda_fail(e, "pack_gate_weights launch");
      packed = wpack;
    }
    cudaError_t e = rgk::launch_rglru_chan(fuse_conv ? xb : c, pos, pos64, p->a_param, p->gate_x_b,
                                           p->gate_a_b, packed, h0, yb, y_activated, B, T, H, out,
                                           h_last, scan_ws, math, s, fuse_conv ? p->conv_w : nullptr,
                                           fuse_conv ? p->conv_b : nullptr);
    if (e != cudaSuccess) return cuda_fail(e, "fused RG-LRU launch");
    return RGK_OK;
  }
  int rc = run_gates(c, pos, pos64, p, B * T, H, bw, dtype,
                     want_fused ? RGK_GATES_AUTO : gates_impl, wpack, a_buf,
                     xn_buf, scan_ws, s);
  if (rc) return rc;
  cudaError_t e = rgk::launch_scan(xn_buf, a_buf, nullptr, nullptr, 0, h0, yb, y_activated, B, T, E,
                                   dtype, out, h_last, scan_ws, s);
  if (e != cudaSuccess) return cuda_fail(e, "scan launch");
  return RGK_OK;
}

// Carves the workspace of the composed calls: [scan scratch | c | a | xn | packed gate weights].
struct PathWs {
  void* scan;
  void* c;
  void* a;
  void* xn;
  void* wpack;
  size_t total;
};

PathWs carve(void* ws, int64_t B, int64_t T, int64_t E, int dtype) {
  PathWs w;
  size_t scan_bytes = rgk::scan_workspace_bytes(B, T, E, dtype);
  const size_t fused_bytes = dtype == RGK_BF16 ? rgk::rglru_chan_workspace_bytes(B, T, E) : 0;
  if (fused_bytes > scan_bytes) scan_bytes = fused_bytes;
  const size_t act = up256(static_cast<size_t>(B) * T * E * elem_size(dtype));
  char* base = static_cast<char*>(ws);
  w.scan = base;
  w.c = base ? base + scan_bytes : nullptr;
  w.a = base ? base + scan_bytes + act : nullptr;
  w.xn = base ? base + scan_bytes + 2 * act : nullptr;
  w.wpack = base ? base + scan_bytes + 3 * act : nullptr;
  // K-major copy of both gate weights for the tensor-core kernels: 2 * E * 256 bfloat16, or for
  // float32 the same split into a high and a low part (2 * 2 * E * 256 float32).
  w.total = scan_bytes + 3 * act + up256(static_cast<size_t>(E) * (dtype == RGK_BF16 ? 1024 : 4096));
  return w;
}

}  // namespace

extern "C" {

int rgk_abi_version(void) { return RGK_ABI_VERSION; }

const char* rgk_last_error(void) { return g_err; }

int rgk_device_check(void) { return device_ok(); }

size_t rgk_workspace_bytes(int64_t B, int64_t T, int64_t E, int dtype) {
  if (B < 0 || T < 0 || E < 0 || (dtype != RGK_F32 && dtype != RGK_BF16)) return 0;
  if (T < 1) T = 1;
  return carve(nullptr, B, T, E, dtype).total;
}

int rgk_workspace_status(void* workspace, void* stream) {
  RGK_REQUIRE(workspace != nullptr, RGK_EINVAL, "workspace is NULL");
  int status = 0;
  RGK_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), "cudaStreamSynchronize");
  RGK_CUDA(cudaMemcpy(&status, workspace, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy");
  if (status == rgk::kStatusBounds) {
    RGK_CUDA(cudaMemset(workspace, 0, sizeof(int)), "cudaMemset");
    return fail(RGK_EBOUNDS, "a range-checked index fell outside its array (checks build); the "
                             "access was skipped and the results are invalid");
  }
  if (status == rgk::kStatusTimeout) {
    // reported once: the word is cleared so that later calls are judged on their own
    RGK_CUDA(cudaMemset(workspace, 0, sizeof(int)), "cudaMemset");
    return fail(RGK_ETIMEOUT, "a bounded device-side wait expired since the status word was last "
                              "cleared; results of the calls on this workspace since then are invalid");
  }
  return RGK_OK;
}

int rgk_set_conv_fusion(int enabled) {
  return g_conv_fusion.exchange(enabled != 0 ? 1 : 0, std::memory_order_relaxed);
}

int rgk_conv1d_prefill(const void* x, const void* segment_pos, int pos_dtype, const void* w,
                       const void* b, int64_t B, int64_t T, int64_t E, int W, int dtype, void* out,
                       void* cache_out, void* stream) {
  int rc = check_common(B, T, E, dtype);
  if (rc) return rc;
  RGK_REQUIRE(W == 4, RGK_ESHAPE, "temporal width %d is not supported (only 4)", W);
  RGK_REQUIRE(pos_dtype == RGK_I32 || pos_dtype == RGK_I64, RGK_EINVAL, "unknown index dtype");
  RGK_REQUIRE(x && segment_pos && w && b && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(w) && aligned16(b) && aligned16(out) && aligned16(cache_out),
              RGK_EALIGN, "pointers must be 16-byte aligned");
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_conv1d_prefill(x, segment_pos, pos_dtype, w, b, B, T, E, dtype, out,
                                      cache_out, static_cast<cudaStream_t>(stream)),
           "conv1d_prefill launch");
  if (T == 0 && cache_out && B * E > 0)
    RGK_CUDA(cudaMemsetAsync(cache_out, 0, (size_t)B * 3 * E * elem_size(dtype),
                             static_cast<cudaStream_t>(stream)), "cudaMemsetAsync");
  return RGK_OK;
}

int rgk_conv1d_decode(const void* x, const void* cache_in, const void* w, const void* b, int64_t B,
                      int64_t E, int W, int dtype, void* out, void* cache_out, void* stream) {
  int rc = check_common(B, 1, E, dtype);
  if (rc) return rc;
  RGK_REQUIRE(W == 4, RGK_ESHAPE, "temporal width %d is not supported (only 4)", W);
  RGK_REQUIRE(x && cache_in && w && b && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(cache_in) && aligned16(w) && aligned16(b) &&
                  aligned16(out) && aligned16(cache_out),
              RGK_EALIGN, "pointers must be 16-byte aligned");
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_conv1d_decode(x, cache_in, w, b, B, E, dtype, out, cache_out,
                                     static_cast<cudaStream_t>(stream)),
           "conv1d_decode launch");
  return RGK_OK;
}

int rgk_blockdiag_linear(const void* x, const void* w, const void* b, int64_t M, int H, int bw,
                         int dtype, void* out, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(M >= 0 && H >= 1 && bw >= 1, RGK_EINVAL, "bad size (M=%lld H=%d bw=%d)", (long long)M,
              H, bw);
  RGK_REQUIRE(bw % 16 == 0, RGK_ESHAPE, "head width %d is not a multiple of 16", bw);
  RGK_REQUIRE(M <= (int64_t)0x7fffffff * 64, RGK_ESHAPE, "too many rows");
  RGK_REQUIRE(x && w && b && out, RGK_EINVAL, "NULL pointer argument");
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_blockdiag_linear_simt(x, w, b, M, H, bw, dtype, out,
                                             static_cast<cudaStream_t>(stream)),
           "blockdiag_linear launch");
  return RGK_OK;
}

int rgk_linear_scan(const void* x, const void* a, const uint8_t* reset, const float* h0,
                    const void* y_mul, int64_t B, int64_t T, int64_t E, int dtype, void* y,
                    float* h_last, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_common(B, T, E, dtype);
  if (rc) return rc;
  RGK_REQUIRE(x && a && y, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(a) && aligned16(y) && aligned16(y_mul) && aligned16(h0) &&
                  aligned16(h_last),
              RGK_EALIGN, "pointers must be 16-byte aligned");
  if (B * T * E == 0) return RGK_OK;
  const size_t need = rgk::scan_workspace_bytes(B, T, E, dtype);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= need, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_scan(x, a, reset, nullptr, 0, h0, y_mul, 0, B, T, E, dtype, y, h_last,
                            workspace, static_cast<cudaStream_t>(stream)),
           "scan launch");
  return RGK_OK;
}

size_t rgk_gate_pack_bytes(int H) { return H > 0 ? rgk::gates_tc_packed_bytes(H) : 0; }

size_t rgk_gate_pack_bytes_for(int H, int dtype) {
  if (H <= 0) return 0;
  if (dtype == RGK_BF16) return rgk::gates_tc_packed_bytes(H);
  if (dtype == RGK_F32) return rgk::gates_tf32_packed_bytes(H);
  return 0;
}

int rgk_pack_gate_weights(const rgk_params* p, int H, int bw, int dtype, void* packed_out,
                          void* stream) {
  int rc = check_params(p, false);
  if (rc) return rc;
  RGK_REQUIRE(H >= 1 && packed_out != nullptr && aligned16(packed_out), RGK_EINVAL,
              "bad H or packed_out");
  RGK_REQUIRE(rgk::gates_tc_supported(dtype, bw, 1) || rgk::gates_tf32_supported(dtype, bw, 1),
              RGK_ESHAPE, "packed gate weights exist for head width 256 only");
  RGK_CHECK_DEVICE();
  if (dtype == RGK_F32) {
    RGK_CUDA(rgk::launch_pack_gate_weights_tf32(p->gate_x_w, p->gate_a_w, H, packed_out,
                                                static_cast<cudaStream_t>(stream)),
             "pack_gate_weights (TF32 split) launch");
    return RGK_OK;
  }
  RGK_CUDA(rgk::launch_pack_gate_weights(p->gate_x_w, p->gate_a_w, H, packed_out,
                                         static_cast<cudaStream_t>(stream)),
           "pack_gate_weights launch");
  return RGK_OK;
}

int rgk_linear_scan_static(const void* x, const void* a, const uint8_t* reset, const float* h0,
                           const void* y_mul, int64_t B, int64_t T, int64_t E, int dtype, void* y,
                           float* h_last, int* status_out, void* stream) {
  int rc = check_common(B, T, E, dtype);
  if (rc) return rc;
  RGK_REQUIRE(x && a && y, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(a) && aligned16(y) && aligned16(y_mul) && aligned16(h0) &&
                  aligned16(h_last),
              RGK_EALIGN, "pointers must be 16-byte aligned");
  if (B * T * E == 0) return RGK_OK;
  const size_t need = rgk::scan_workspace_bytes(B, T, E, dtype);
  const size_t have = rgk::scan_static_scratch_bytes();
  RGK_REQUIRE(need <= have, RGK_ESHAPE,
              "problem needs %zu bytes of scan scratch but the built-in scratch holds %zu; use "
              "rgk_linear_scan with a caller workspace for sizes this large", need, have);
  RGK_CHECK_DEVICE();
  void* scratch = nullptr;
  RGK_CUDA(rgk::scan_static_scratch(&scratch), "cudaGetSymbolAddress(built-in scan scratch)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left: the status word is cleared here, the ticket
  // and the look-back flags by the launch below; records are rewritten before they are read.
  RGK_CUDA(cudaMemsetAsync(scratch, 0, sizeof(int), s), "cudaMemsetAsync");
  RGK_CUDA(rgk::launch_scan(x, a, reset, nullptr, 0, h0, y_mul, 0, B, T, E, dtype, y, h_last, scratch,
                            s),
           "scan launch");
  if (status_out != nullptr)
    RGK_CUDA(cudaMemcpyAsync(status_out, scratch, sizeof(int), cudaMemcpyDeviceToDevice, s),
             "cudaMemcpyAsync");
  return RGK_OK;
}

int rgk_selftest_wait_expiry(void* workspace, size_t workspace_bytes, void* stream) {
  // A scan over 2 sequences x 3 time tiles x 64 channels whose first time tile is never launched:
  // the tiles of the second time tile look back for records nobody publishes, give up after 200
  // polls (tens of microseconds), raise the status word, take a zero carry and finish.
  const int64_t B = 2, T = 3 * 128, E = 64;
  const size_t act = static_cast<size_t>(B * T * E) * 2;
  const size_t need = up256(rgk::scan_workspace_bytes(B, T, E, RGK_BF16)) + 3 * up256(act);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= need, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  RGK_CHECK_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(workspace);
  char* x = base + up256(rgk::scan_workspace_bytes(B, T, E, RGK_BF16));
  char* a = x + up256(act);
  char* y = a + up256(act);
  RGK_CUDA(cudaMemsetAsync(x, 0, 3 * up256(act), s), "cudaMemsetAsync");
  RGK_CUDA(rgk::launch_scan(x, a, nullptr, nullptr, 0, nullptr, nullptr, 0, B, T, E, RGK_BF16, y,
                            nullptr, workspace, s, /*skip_time_tiles=*/1, /*spin_limit=*/200),
           "scan launch");
  return RGK_OK;
}

int rgk_rglru_forward(const void* x, const void* segment_pos, int pos_dtype, const rgk_params* p,
                      const float* h0, int64_t B, int64_t T, int64_t E, int H, int dtype,
                      int gates_impl, void* y, float* h_last, void* workspace,
                      size_t workspace_bytes, void* stream) {
  int rc = check_common(B, T, E, dtype);
  if (rc) return rc;
  if ((rc = check_heads(E, H))) return rc;
  if ((rc = check_params(p, false))) return rc;
  RGK_REQUIRE(pos_dtype == RGK_I32 || pos_dtype == RGK_I64, RGK_EINVAL, "unknown index dtype");
  RGK_REQUIRE(gates_impl >= RGK_GATES_AUTO && gates_impl <= RGK_GATES_FUSED_EXACT, RGK_EINVAL,
              "unknown gates_impl %d", gates_impl);
  RGK_REQUIRE(x && segment_pos && y, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(y) && aligned16(h0) && aligned16(h_last), RGK_EALIGN,
              "pointers must be 16-byte aligned");
  if (B * T * E == 0) return RGK_OK;
  const PathWs w = carve(workspace, B, T, E, dtype);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= w.total, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", w.total, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  RGK_CHECK_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bw = (int)(E / H);
  (void)bw;
  return run_rglru(x, segment_pos, pos_dtype, p, h0, nullptr, 0, B, T, E, H, dtype, gates_impl,
                   w.wpack, w.a, w.xn, w.scan, y, h_last, s);
}

int rgk_recurrent_path_prefill(const void* xb, const void* yb, const void* segment_pos,
                               int pos_dtype, const rgk_params* p, const float* h0, int64_t B,
                               int64_t T, int64_t E, int H, int W, int dtype, int gates_impl,
                               void* out, float* h_last, void* conv_cache_out, void* workspace,
                               size_t workspace_bytes, void* stream) {
  int rc = check_common(B, T, E, dtype);
  if (rc) return rc;
  if ((rc = check_heads(E, H))) return rc;
  if ((rc = check_params(p, true))) return rc;
  RGK_REQUIRE(W == 4, RGK_ESHAPE, "temporal width %d is not supported (only 4)", W);
  RGK_REQUIRE(pos_dtype == RGK_I32 || pos_dtype == RGK_I64, RGK_EINVAL, "unknown index dtype");
  RGK_REQUIRE(gates_impl >= RGK_GATES_AUTO && gates_impl <= RGK_GATES_FUSED_EXACT, RGK_EINVAL,
              "unknown gates_impl %d", gates_impl);
  RGK_REQUIRE(xb && segment_pos && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(xb) && aligned16(yb) && aligned16(out) && aligned16(h0) &&
                  aligned16(h_last) && aligned16(conv_cache_out),
              RGK_EALIGN, "pointers must be 16-byte aligned");
  RGK_REQUIRE(T >= 1 || B * E == 0, RGK_ESHAPE, "prefill needs at least one token");
  if (B * T * E == 0) return RGK_OK;
  const PathWs w = carve(workspace, B, T, E, dtype);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= w.total, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", w.total, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  RGK_CHECK_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bw = (int)(E / H);
  (void)bw;
  return run_rglru(w.c, segment_pos, pos_dtype, p, h0, yb, 0, B, T, E, H, dtype, gates_impl,
                   w.wpack, w.a, w.xn, w.scan, out, h_last, s, xb, conv_cache_out);
}

int rgk_dense_linear(const void* x, const void* weight, const void* bias, int64_t M, int64_t K,
                     int64_t N, int dtype, int act, void* out, int* status, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(act == RGK_ACT_NONE || act == RGK_ACT_GELU_TANH, RGK_EINVAL, "unknown act %d", act);
  RGK_REQUIRE(M >= 0 && K >= 1 && N >= 1, RGK_EINVAL, "bad size (M=%lld K=%lld N=%lld)",
              (long long)M, (long long)K, (long long)N);
  RGK_REQUIRE(x && weight && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(out) && aligned16(bias), RGK_EALIGN,
              "pointers must be 16-byte aligned");
  RGK_REQUIRE(rgk::dense_tc_supported(dtype, M > 0 ? M : 1, K, N), RGK_ESHAPE,
              "the tensor-core linear covers bfloat16 with K and N multiples of 8 "
              "(dtype %d, K=%lld, N=%lld)", dtype, (long long)K, (long long)N);
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_dense_tc(x, weight, bias, nullptr, M, (int)K, (int)N, act == RGK_ACT_GELU_TANH, out,
                                status, static_cast<cudaStream_t>(stream)),
           "dense linear launch");
  return RGK_OK;
}

int rgk_dense_linear_small(const void* x, const void* weight, const void* bias, const void* residual,
                           int64_t M, int64_t K, int64_t N, int dtype, int act, void* out,
                           int* status, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(act == RGK_ACT_NONE || act == RGK_ACT_GELU_TANH || act == RGK_ACT_GEGLU, RGK_EINVAL,
              "unknown act %d", act);
  RGK_REQUIRE(M >= 0 && K >= 1 && N >= 1, RGK_EINVAL, "bad size (M=%lld K=%lld N=%lld)",
              (long long)M, (long long)K, (long long)N);
  RGK_REQUIRE(x && weight && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(act != RGK_ACT_GEGLU || (residual == nullptr && bias != nullptr && N % 128 == 0),
              RGK_ESHAPE, "GeGLU takes the packed up-projection with its bias (N = 2 X with X a "
              "multiple of 64, N=%lld) and no residual", (long long)N);
  RGK_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(out) && aligned16(bias) &&
              aligned16(residual), RGK_EALIGN, "pointers must be 16-byte aligned");
  RGK_REQUIRE(rgk::dense_small_supported(dtype, M > 0 ? M : 1, K, N), RGK_ESHAPE,
              "the few-row linear covers bfloat16 with M <= 256 and K and N multiples of 8 "
              "(dtype %d, M=%lld, K=%lld, N=%lld)", dtype, (long long)M, (long long)K, (long long)N);
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_dense_small(x, weight, bias, nullptr, nullptr, residual, M, (int)K, (int)N, 0,
                                   act, out, nullptr, status, static_cast<cudaStream_t>(stream)),
           "few-row dense linear launch");
  return RGK_OK;
}

int rgk_dense_linear_small_pair(const void* x, const void* weight_a, const void* bias_a,
                                const void* weight_b, const void* bias_b, int64_t M, int64_t K,
                                int64_t N_a, int64_t N_b, int dtype, void* out_a, void* out_b,
                                int* status, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(M >= 0 && K >= 1 && N_a >= 1 && N_b >= 1, RGK_EINVAL,
              "bad size (M=%lld K=%lld N_a=%lld N_b=%lld)", (long long)M, (long long)K,
              (long long)N_a, (long long)N_b);
  RGK_REQUIRE(x && weight_a && weight_b && out_a && out_b, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(weight_a) && aligned16(weight_b) && aligned16(out_a) &&
              aligned16(out_b) && aligned16(bias_a) && aligned16(bias_b), RGK_EALIGN,
              "pointers must be 16-byte aligned");
  RGK_REQUIRE(rgk::dense_small_supported(dtype, M > 0 ? M : 1, K, N_a + N_b) && N_a % 128 == 0 &&
              N_b % 8 == 0, RGK_ESHAPE,
              "the paired few-row linear covers bfloat16 with M <= 256, K and N_b multiples of 8 and "
              "N_a a multiple of 128 (dtype %d, M=%lld, K=%lld, N_a=%lld, N_b=%lld)", dtype,
              (long long)M, (long long)K, (long long)N_a, (long long)N_b);
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_dense_small(x, weight_a, bias_a, weight_b, bias_b, nullptr, M, (int)K, (int)N_a,
                                   (int)N_b, 0, out_a, out_b, status, static_cast<cudaStream_t>(stream)),
           "paired few-row dense linear launch");
  return RGK_OK;
}

int rgk_embed(const void* tokens, int token_dtype, const void* table, int64_t M, int64_t V,
              int64_t D, float scale, int dtype, void* out, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(token_dtype == RGK_I32 || token_dtype == RGK_I64, RGK_EINVAL,
              "unknown token dtype %d", token_dtype);
  RGK_REQUIRE(M >= 0 && V >= 1 && D >= 1, RGK_EINVAL, "bad size (M=%lld V=%lld D=%lld)",
              (long long)M, (long long)V, (long long)D);
  RGK_REQUIRE(tokens && table && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(table) && aligned16(out), RGK_EALIGN, "pointers must be 16-byte aligned");
  RGK_REQUIRE((D * (int64_t)elem_size(dtype)) % 16 == 0, RGK_ESHAPE,
              "the embedding width must be a multiple of a 16-byte pack (D=%lld)", (long long)D);
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_embed(tokens, token_dtype == RGK_I64, table, M, V, D, scale, dtype, out,
                             static_cast<cudaStream_t>(stream)),
           "embed launch");
  return RGK_OK;
}

int rgk_logits(const void* x, const void* table, int64_t M, int64_t D, int64_t V, float cap,
               int dtype, void* out, int* status, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(M >= 0 && D >= 1 && V >= 1, RGK_EINVAL, "bad size (M=%lld D=%lld V=%lld)",
              (long long)M, (long long)D, (long long)V);
  RGK_REQUIRE(cap >= 0.0f, RGK_EINVAL, "the soft cap must not be negative");
  RGK_REQUIRE(x && table && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(table) && aligned16(out), RGK_EALIGN,
              "pointers must be 16-byte aligned");
  RGK_REQUIRE(rgk::dense_tc_supported(dtype, M > 0 ? M : 1, D, V), RGK_ESHAPE,
              "the tensor-core logits cover bfloat16 with D and V multiples of 8 "
              "(dtype %d, D=%lld, V=%lld)", dtype, (long long)D, (long long)V);
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_dense_tc(x, table, nullptr, nullptr, M, (int)D, (int)V, 0, out, status,
                                static_cast<cudaStream_t>(stream), cap),
           "logits launch");
  return RGK_OK;
}

int rgk_argmax(const void* x, int64_t M, int64_t V, int dtype, int* out, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(M >= 0 && V >= 1 && V < ((int64_t)1 << 31), RGK_EINVAL, "bad size (M=%lld V=%lld)",
              (long long)M, (long long)V);
  RGK_REQUIRE(x && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x), RGK_EALIGN, "pointers must be 16-byte aligned");
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_argmax(x, M, V, dtype, out, static_cast<cudaStream_t>(stream)),
           "argmax launch");
  return RGK_OK;
}

int rgk_geglu_bias(const void* up, const void* bias, int64_t M, int64_t X, int dtype, void* out,
                   void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(M >= 0 && X >= 1, RGK_EINVAL, "bad size (M=%lld X=%lld)", (long long)M, (long long)X);
  RGK_REQUIRE(up && bias && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(up) && aligned16(bias) && aligned16(out), RGK_EALIGN,
              "pointers must be 16-byte aligned");
  RGK_REQUIRE((X * (int64_t)elem_size(dtype)) % 16 == 0, RGK_ESHAPE,
              "the expanded width must be a multiple of a 16-byte pack (X=%lld)", (long long)X);
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_geglu_bias(up, bias, M, X, dtype, out, static_cast<cudaStream_t>(stream)),
           "geglu launch");
  return RGK_OK;
}

size_t rgk_block_workspace_bytes(int64_t B, int64_t T, int64_t D, int64_t E, int dtype) {
  if (B < 0 || T < 0 || D < 0 || E < 0 || (dtype != RGK_F32 && dtype != RGK_BF16)) return 0;
  if (T < 1) T = 1;
  const size_t act = up256(static_cast<size_t>(B) * T * E * elem_size(dtype));
  return carve(nullptr, B, T, E, dtype).total + 2 * act;
}

// Validation and launches shared by the block entry points.  x_in is what linear_x / linear_y read
// (the block input, or its RMSNorm), residual (may be NULL) is added to linear_out's result, `ws` is
// a block workspace.
static int block_prefill_impl(const void* x_in, const void* residual, const void* segment_pos,
                              int pos_dtype, const rgk_block_params* p, int64_t B, int64_t T,
                              int64_t D, int64_t E, int H, int dtype, void* out, float* h_last,
                              void* conv_cache_out, void* workspace, cudaStream_t s) {
  const PathWs w = carve(workspace, B, T, E, dtype);
  const size_t act = up256(static_cast<size_t>(B) * T * E * elem_size(dtype));
  char* xb = static_cast<char*>(workspace) + w.total;   // later reused for the joined output
  char* yb = xb + act;
  int* status = static_cast<int*>(workspace);
  const int64_t M = B * T;
  int rc;
  // y branch with its gelu in the GEMM epilogue, x branch plain
  RGK_CUDA(rgk::launch_dense_tc(x_in, p->linear_y_w, p->linear_y_b, nullptr, M, (int)D, (int)E, 1, yb,
                                status, s),
           "linear_y launch");
  RGK_CUDA(rgk::launch_dense_tc(x_in, p->linear_x_w, p->linear_x_b, nullptr, M, (int)D, (int)E, 0, xb,
                                status, s),
           "linear_x launch");
  // Conv1D inside the RG-LRU kernel where that kernel applies (the joined output y * gelu(yb) then
  // goes to the conv-output buffer, which the fused form does not use), else as its own kernel
  // (a warp reads its tile of yb before it writes the same tile of the output); with a separate
  // conv kernel xb has been consumed by then and receives the output
  const bool fused = rgk::rglru_chan_supported(dtype, (int)(E / H), B, T) && conv_fusion_enabled();
  char* joined = fused ? yb : xb;
  if ((rc = run_rglru(w.c, segment_pos, pos_dtype, &p->path, nullptr, yb, 1, B, T, E, H, dtype,
                      RGK_GATES_AUTO, w.wpack, w.a, w.xn, w.scan, joined, h_last, s, xb,
                      conv_cache_out)))
    return rc;
  RGK_CUDA(rgk::launch_dense_tc(joined, p->linear_out_w, p->linear_out_b, residual, M, (int)E, (int)D,
                                0, out, status, s),
           "linear_out launch");
  return RGK_OK;
}

static int check_block_args(const void* x, const void* segment_pos, int pos_dtype,
                            const rgk_block_params* p, int64_t B, int64_t T, int64_t D, int64_t E,
                            int H, int W, int dtype, const void* out, const float* h_last,
                            const void* conv_cache_out) {
  int rc = check_common(B, T, E, dtype);
  if (rc) return rc;
  if ((rc = check_heads(E, H))) return rc;
  RGK_REQUIRE(p != nullptr, RGK_EINVAL, "params is NULL");
  if ((rc = check_params(&p->path, true))) return rc;
  RGK_REQUIRE(p->linear_y_w && p->linear_x_w && p->linear_out_w, RGK_EINVAL,
              "a linear weight pointer is NULL");
  RGK_REQUIRE(aligned16(p->linear_y_w) && aligned16(p->linear_x_w) && aligned16(p->linear_out_w) &&
                  aligned16(p->linear_y_b) && aligned16(p->linear_x_b) && aligned16(p->linear_out_b),
              RGK_EALIGN, "parameter pointers must be 16-byte aligned");
  RGK_REQUIRE(W == 4, RGK_ESHAPE, "temporal width %d is not supported (only 4)", W);
  RGK_REQUIRE(pos_dtype == RGK_I32 || pos_dtype == RGK_I64, RGK_EINVAL, "unknown index dtype");
  RGK_REQUIRE(x && segment_pos && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(out) && aligned16(h_last) && aligned16(conv_cache_out),
              RGK_EALIGN, "pointers must be 16-byte aligned");
  RGK_REQUIRE(D >= 8 && D % 8 == 0, RGK_ESHAPE, "block width %lld is not a multiple of 8",
              (long long)D);
  const int bw = (int)(E / H);
  RGK_REQUIRE(rgk::gates_tc_supported(dtype, bw, B * T > 0 ? B * T : 1), RGK_ESHAPE,
              "the fused block covers bfloat16 with head width 256 only (dtype %d, head width %d)",
              dtype, bw);
  return RGK_OK;
}

int rgk_recurrent_block_prefill(const void* x, const void* segment_pos, int pos_dtype,
                                const rgk_block_params* p, int64_t B, int64_t T, int64_t D,
                                int64_t E, int H, int W, int dtype, void* out, float* h_last,
                                void* conv_cache_out, void* workspace, size_t workspace_bytes,
                                void* stream) {
  int rc = check_block_args(x, segment_pos, pos_dtype, p, B, T, D, E, H, W, dtype, out, h_last,
                            conv_cache_out);
  if (rc) return rc;
  if (B * T * E == 0) return RGK_OK;
  const size_t need = rgk_block_workspace_bytes(B, T, D, E, dtype);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= need, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  RGK_CHECK_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return block_prefill_impl(x, nullptr, segment_pos, pos_dtype, p, B, T, D, E, H, dtype, out, h_last,
                            conv_cache_out, workspace, s);
}

int rgk_rmsnorm(const void* x, const void* scale, int64_t M, int64_t D, float eps, int dtype,
                void* out, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(M >= 0 && D >= 1, RGK_EINVAL, "bad size (M=%lld D=%lld)", (long long)M, (long long)D);
  RGK_REQUIRE(x && scale && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(scale) && aligned16(out), RGK_EALIGN,
              "pointers must be 16-byte aligned");
  RGK_REQUIRE(rgk::rmsnorm_supported(dtype, D), RGK_ESHAPE,
              "RMSNorm covers widths that are multiples of a 16-byte pack, up to 1024 packs "
              "(dtype %d, D=%lld)", dtype, (long long)D);
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_rmsnorm(x, scale, M, D, eps, dtype, out, static_cast<cudaStream_t>(stream)),
           "rmsnorm launch");
  return RGK_OK;
}

int rgk_add_rmsnorm(const void* a, const void* b, const void* scale, int64_t M, int64_t D, float eps,
                    int dtype, void* sum_out, void* out, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(M >= 0 && D >= 1, RGK_EINVAL, "bad size (M=%lld D=%lld)", (long long)M, (long long)D);
  RGK_REQUIRE(a && b && scale && sum_out && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(a) && aligned16(b) && aligned16(scale) && aligned16(sum_out) && aligned16(out),
              RGK_EALIGN, "pointers must be 16-byte aligned");
  RGK_REQUIRE(rgk::rmsnorm_supported(dtype, D), RGK_ESHAPE,
              "RMSNorm covers widths that are multiples of a 16-byte pack, up to 1024 packs "
              "(dtype %d, D=%lld)", dtype, (long long)D);
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_rmsnorm(a, scale, M, D, eps, dtype, out, static_cast<cudaStream_t>(stream), b,
                               sum_out),
           "add + rmsnorm launch");
  return RGK_OK;
}

size_t rgk_residual_workspace_bytes(int64_t B, int64_t T, int64_t D, int64_t E, int dtype) {
  const size_t block = rgk_block_workspace_bytes(B, T, D, E, dtype);
  if (block == 0) return 0;
  if (T < 1) T = 1;
  return block + up256(static_cast<size_t>(B) * T * D * elem_size(dtype));
}

int rgk_residual_block_prefill(const void* x, const void* segment_pos, int pos_dtype,
                               const rgk_block_params* p, const void* norm_scale, float eps,
                               int64_t B, int64_t T, int64_t D, int64_t E, int H, int W, int dtype,
                               void* out, float* h_last, void* conv_cache_out, void* workspace,
                               size_t workspace_bytes, void* stream) {
  int rc = check_block_args(x, segment_pos, pos_dtype, p, B, T, D, E, H, W, dtype, out, h_last,
                            conv_cache_out);
  if (rc) return rc;
  RGK_REQUIRE(norm_scale != nullptr, RGK_EINVAL, "norm_scale is NULL");
  RGK_REQUIRE(aligned16(norm_scale), RGK_EALIGN, "norm_scale must be 16-byte aligned");
  RGK_REQUIRE(rgk::rmsnorm_supported(dtype, D), RGK_ESHAPE, "block width %lld is not covered by the "
              "RMSNorm kernel", (long long)D);
  if (B * T * E == 0) return RGK_OK;
  const size_t block = rgk_block_workspace_bytes(B, T, D, E, dtype);
  const size_t need = rgk_residual_workspace_bytes(B, T, D, E, dtype);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= need, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  RGK_CHECK_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* xn = static_cast<char*>(workspace) + block;      // temporal_pre_norm(x)
  RGK_CUDA(rgk::launch_rmsnorm(x, norm_scale, B * T, D, eps, dtype, xn, s), "rmsnorm launch");
  return block_prefill_impl(xn, x, segment_pos, pos_dtype, p, B, T, D, E, H, dtype, out, h_last,
                            conv_cache_out, workspace, s);
}

// ---- MLP block and the channel half of the residual block --------------------------------------

static size_t mlp_pack_w_bytes(int64_t D, int64_t X) { return up256(static_cast<size_t>(2 * X) * D * 2); }

size_t rgk_mlp_pack_bytes(int64_t D, int64_t X) {
  if (D < 8 || X < 64 || D % 8 != 0 || X % 64 != 0) return 0;
  return mlp_pack_w_bytes(D, X) + up256(static_cast<size_t>(2 * X) * 2);
}

int rgk_pack_mlp_up(const void* w, const void* b, int64_t D, int64_t X, int dtype, void* packed_out,
                    void* stream) {
  RGK_REQUIRE(dtype == RGK_BF16, RGK_ESHAPE, "the packed MLP weights are bfloat16 only (dtype %d)",
              dtype);
  RGK_REQUIRE(w && b && packed_out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(D >= 8 && D % 8 == 0 && X >= 64 && X % 64 == 0 && D < (1 << 24) && X < (1 << 23),
              RGK_ESHAPE, "the MLP kernels cover widths that are multiples of 8 and expanded widths "
              "that are multiples of 64 (D=%lld, X=%lld)", (long long)D, (long long)X);
  RGK_REQUIRE(aligned16(w) && aligned16(b) && aligned16(packed_out), RGK_EALIGN,
              "pointers must be 16-byte aligned");
  RGK_CHECK_DEVICE();
  char* out = static_cast<char*>(packed_out);
  RGK_CUDA(rgk::launch_pack_mlp_up(w, b, (int)D, (int)X, out, out + mlp_pack_w_bytes(D, X),
                                   static_cast<cudaStream_t>(stream)),
           "pack_mlp_up launch");
  return RGK_OK;
}

size_t rgk_mlp_workspace_bytes(int64_t M, int64_t D, int64_t X, int dtype) {
  if (M < 0 || D < 1 || X < 1 || dtype != RGK_BF16) return 0;
  if (M < 1) M = 1;
  return 256 + up256(static_cast<size_t>(M) * X * 2) + up256(static_cast<size_t>(M) * D * 2);
}

// out = ffw_down(gelu(up_0) * up_1) [+ residual]; x_in is the MLP's input.
static int mlp_impl(const void* x_in, const void* packed_up, const void* down_w, const void* down_b,
                    const void* residual, int64_t M, int64_t D, int64_t X, void* out,
                    void* workspace, cudaStream_t s) {
  int* status = static_cast<int*>(workspace);
  char* act = static_cast<char*>(workspace) + 256;
  const char* pw = static_cast<const char*>(packed_up);
  RGK_CUDA(rgk::launch_dense_tc(x_in, pw, pw + mlp_pack_w_bytes(D, X), nullptr, M, (int)D,
                                (int)(2 * X), 2, act, status, s),
           "ffw_up launch");
  RGK_CUDA(rgk::launch_dense_tc(act, down_w, down_b, residual, M, (int)X, (int)D, 0, out, status, s),
           "ffw_down launch");
  return RGK_OK;
}

static int check_mlp_args(const void* x, const void* packed_up, const void* down_w,
                          const void* down_b, int64_t M, int64_t D, int64_t X, int dtype,
                          const void* out, const void* workspace, size_t workspace_bytes) {
  RGK_REQUIRE(dtype == RGK_BF16, RGK_ESHAPE, "the MLP kernels are bfloat16 only (dtype %d)", dtype);
  RGK_REQUIRE(M >= 0 && M < ((int64_t)1 << 31), RGK_EINVAL, "bad row count %lld", (long long)M);
  RGK_REQUIRE(D >= 8 && D % 8 == 0 && X >= 64 && X % 64 == 0 && D < (1 << 24) && X < (1 << 23),
              RGK_ESHAPE, "the MLP kernels cover widths that are multiples of 8 and expanded widths "
              "that are multiples of 64 (D=%lld, X=%lld)", (long long)D, (long long)X);
  RGK_REQUIRE(x && packed_up && down_w && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(x) && aligned16(packed_up) && aligned16(down_w) && aligned16(down_b) &&
                  aligned16(out),
              RGK_EALIGN, "pointers must be 16-byte aligned");
  if (M == 0) return RGK_OK;
  const size_t need = rgk_mlp_workspace_bytes(M, D, X, dtype);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= need, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  return RGK_OK;
}

int rgk_mlp_block(const void* x, const void* packed_up, const void* down_w, const void* down_b,
                  const void* residual, int64_t M, int64_t D, int64_t X, int dtype, void* out,
                  void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_mlp_args(x, packed_up, down_w, down_b, M, D, X, dtype, out, workspace,
                          workspace_bytes);
  if (rc) return rc;
  RGK_REQUIRE(aligned16(residual), RGK_EALIGN, "pointers must be 16-byte aligned");
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return mlp_impl(x, packed_up, down_w, down_b, residual, M, D, X, out, workspace, s);
}

int rgk_residual_channel(const void* residual_in, const void* norm_scale, float eps,
                         const void* packed_up, const void* down_w, const void* down_b, int64_t M,
                         int64_t D, int64_t X, int dtype, void* out, void* workspace,
                         size_t workspace_bytes, void* stream) {
  int rc = check_mlp_args(residual_in, packed_up, down_w, down_b, M, D, X, dtype, out, workspace,
                          workspace_bytes);
  if (rc) return rc;
  RGK_REQUIRE(norm_scale != nullptr, RGK_EINVAL, "norm_scale is NULL");
  RGK_REQUIRE(aligned16(norm_scale), RGK_EALIGN, "norm_scale must be 16-byte aligned");
  RGK_REQUIRE(rgk::rmsnorm_supported(dtype, D), RGK_ESHAPE, "block width %lld is not covered by the "
              "RMSNorm kernel", (long long)D);
  if (M == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* xn = static_cast<char*>(workspace) + 256 + up256(static_cast<size_t>(M) * X * 2);
  RGK_CUDA(rgk::launch_rmsnorm(residual_in, norm_scale, M, D, eps, dtype, xn, s), "rmsnorm launch");
  return mlp_impl(xn, packed_up, down_w, down_b, residual_in, M, D, X, out, workspace, s);
}

// ---- local attention ----------------------------------------------------------------------------

int rgk_rope(void* x, const void* segment_pos, int pos_dtype, int64_t rows, int heads, int head_dim,
             int dtype, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(pos_dtype == RGK_I32 || pos_dtype == RGK_I64, RGK_EINVAL, "unknown index dtype");
  RGK_REQUIRE(rows >= 0 && heads >= 1 && head_dim >= 4 && head_dim % 4 == 0, RGK_EINVAL,
              "bad size (rows=%lld heads=%d head_dim=%d)", (long long)rows, heads, head_dim);
  RGK_REQUIRE(x && segment_pos, RGK_EINVAL, "NULL pointer argument");
  if (rows == 0) return RGK_OK;
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_rope(x, segment_pos, pos_dtype == RGK_I64, rows, heads, head_dim, dtype,
                            static_cast<cudaStream_t>(stream)),
           "rope launch");
  return RGK_OK;
}

size_t rgk_attention_workspace_bytes(int64_t B, int64_t T) {
  if (B < 0 || T < 0) return 0;
  return rgk::attention_workspace_bytes(B < 1 ? 1 : B, T < 1 ? 1 : T);
}

int rgk_local_attention_prefill(const void* q, const void* k, const void* v, const void* segment_pos,
                                int pos_dtype, int64_t B, int64_t T, int N, int head_dim, int window,
                                int dtype, void* out, void* workspace, size_t workspace_bytes,
                                void* stream) {
  RGK_REQUIRE(pos_dtype == RGK_I32 || pos_dtype == RGK_I64, RGK_EINVAL, "unknown index dtype");
  RGK_REQUIRE(B >= 0 && T >= 0 && N >= 1 && window >= 1, RGK_EINVAL, "bad size");
  RGK_REQUIRE(q && k && v && segment_pos && out, RGK_EINVAL, "NULL pointer argument");
  RGK_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), RGK_EALIGN,
              "pointers must be 16-byte aligned");
  RGK_REQUIRE(rgk::attention_supported(dtype, head_dim, B > 0 ? B : 1, T > 0 ? T : 1, N), RGK_ESHAPE,
              "the attention kernel covers bfloat16 with head dimension 256 (dtype %d, head_dim %d)",
              dtype, head_dim);
  if (B * T == 0) return RGK_OK;
  const size_t need = rgk_attention_workspace_bytes(B, T);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= need, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  RGK_CHECK_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RGK_CUDA(rgk::launch_attention_prefill(q, k, v, segment_pos, pos_dtype == RGK_I64, B, T, N, window,
                                         out, workspace, s),
           "attention launch");
  return RGK_OK;
}

size_t rgk_attention_decode_workspace_bytes(int64_t B, int N, int window) {
  if (B < 0 || N < 1 || window < 1) return 0;
  return rgk::attention_decode_workspace_bytes(B < 1 ? 1 : B, N, window);
}

int rgk_local_attention_decode(const void* q, const void* k_new, const void* v_new, void* keys,
                               void* values, int* num_tokens, int64_t B, int N, int head_dim,
                               int window, int dtype, int update, void* out, void* workspace,
                               size_t workspace_bytes, void* stream) {
  RGK_REQUIRE(dtype == RGK_F32 || dtype == RGK_BF16, RGK_EINVAL, "unknown dtype %d", dtype);
  RGK_REQUIRE(B >= 0 && N >= 1 && window >= 1, RGK_EINVAL, "bad size");
  RGK_REQUIRE(q && k_new && v_new && keys && values && num_tokens && out, RGK_EINVAL,
              "NULL pointer argument");
  RGK_REQUIRE(aligned16(q) && aligned16(k_new) && aligned16(v_new) && aligned16(keys) &&
                  aligned16(values) && aligned16(out), RGK_EALIGN,
              "pointers must be 16-byte aligned");
  RGK_REQUIRE(rgk::attention_decode_supported(head_dim, N, window), RGK_ESHAPE,
              "the decode attention kernel covers head dimension 256 and 1/2/4/8/10 query heads "
              "(head_dim %d, heads %d, window %d)",
              head_dim, N, window);
  if (B == 0) return RGK_OK;
  const size_t need = rgk_attention_decode_workspace_bytes(B, N, window);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= need, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  RGK_CHECK_DEVICE();
  RGK_CUDA(rgk::launch_attention_decode(q, k_new, v_new, keys, values, num_tokens, B, N, window,
                                        dtype, update, out, workspace,
                                        static_cast<cudaStream_t>(stream)),
           "decode attention launch");
  return RGK_OK;
}

int rgk_recurrent_path_decode(const void* xb, const void* yb, const void* segment_pos,
                              int pos_dtype, const rgk_params* p, const float* h_in,
                              const void* conv_cache_in, int64_t B, int64_t E, int H, int W,
                              int dtype, int gates_impl, void* out, float* h_out,
                              void* conv_cache_out, void* workspace, size_t workspace_bytes,
                              void* stream) {
  int rc = check_common(B, 1, E, dtype);
  if (rc) return rc;
  if ((rc = check_heads(E, H))) return rc;
  if ((rc = check_params(p, true))) return rc;
  RGK_REQUIRE(W == 4, RGK_ESHAPE, "temporal width %d is not supported (only 4)", W);
  RGK_REQUIRE(pos_dtype == RGK_I32 || pos_dtype == RGK_I64, RGK_EINVAL, "unknown index dtype");
  RGK_REQUIRE(gates_impl >= RGK_GATES_AUTO && gates_impl <= RGK_GATES_FUSED_EXACT, RGK_EINVAL,
              "unknown gates_impl %d", gates_impl);
  RGK_REQUIRE(xb && segment_pos && h_in && conv_cache_in && out && h_out, RGK_EINVAL,
              "NULL pointer argument");
  RGK_REQUIRE(aligned16(xb) && aligned16(yb) && aligned16(out) && aligned16(h_in) &&
                  aligned16(h_out) && aligned16(conv_cache_in) && aligned16(conv_cache_out),
              RGK_EALIGN, "pointers must be 16-byte aligned");
  if (B * E == 0) return RGK_OK;
  const PathWs w = carve(workspace, B, 1, E, dtype);
  RGK_REQUIRE(workspace != nullptr && workspace_bytes >= w.total, RGK_EWORKSPACE,
              "workspace of %zu bytes needed, %zu given", w.total, workspace_bytes);
  RGK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RGK_EALIGN,
              "workspace must be 256-byte aligned");
  RGK_CHECK_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bw = (int)(E / H);
  if (gates_impl != RGK_GATES_SIMT && rgk::gates_tc_supported(dtype, bw, B)) {
    // The whole step in one kernel, and nothing else on the stream: a decode loop is one launch
    // per layer.  The states may be updated in place: every element of h and of the conv cache is read and
    // then written by one and the same thread.
    const void* packed = p->gates_packed;
    if (packed == nullptr) {
      RGK_CUDA(rgk::launch_pack_gate_weights(p->gate_x_w, p->gate_a_w, H, w.wpack, s),
               "pack_gate_weights launch");
      packed = w.wpack;
    }
    RGK_CUDA(rgk::launch_path_decode_tc(xb, yb, segment_pos, pos_dtype, p->conv_w, p->conv_b,
                                        p->a_param, p->gate_x_b, p->gate_a_b, packed, h_in,
                                        conv_cache_in, B, H, out, h_out, conv_cache_out, workspace,
                                        s, (gates_impl == RGK_GATES_FUSED_EXACT ||
                                            gates_impl == RGK_GATES_TCGEN05) ? rgk::kMathExact
                                                                             : rgk::kMathFast),
             "fused decode launch");
    return RGK_OK;
  }
  RGK_CUDA(rgk::launch_conv1d_decode(xb, conv_cache_in, p->conv_w, p->conv_b, B, E, dtype, w.c,
                                     conv_cache_out, s),
           "conv1d_decode launch");
  if ((rc = run_gates(w.c, segment_pos, pos_dtype, p, B, H, bw, dtype, gates_impl, w.wpack, w.a,
                      w.xn, workspace, s)))
    return rc;
  RGK_CUDA(rgk::launch_decode_update(w.a, w.xn, h_in, yb, B, E, dtype, out, h_out, s),
           "decode_update launch");
  return RGK_OK;
}

}  // extern "C"
