// C ABI of libb2q.so: argument validation and kernel selection.  Nothing here
// allocates or synchronises; every launch goes to the caller's stream.
#include "common.cuh"
#include "smallm.cuh"
#include "umma_gemm.cuh"
#include "peer_reduce.cuh"

namespace b2q {

ThreadState& tls() {
  static thread_local ThreadState s;
  return s;
}

// implemented in dequant.cu / moe_aux.cu
int dequant_int4(const void*, int, const void*, int, void*, int, int64_t, int64_t, int, cudaStream_t);
int dequant_fp8(const void*, int, const void*, int, int, void*, int, int64_t, int64_t, cudaStream_t);
int moe_topk(const void*, int, int64_t, int, int, int, void*, int, int32_t*, cudaStream_t);
size_t moe_route_workspace_bytes(int64_t, int);
int moe_route(const int32_t*, int64_t, int, int32_t*, int32_t*, int32_t*, int32_t*, void*, cudaStream_t);
int moe_build_tiles(const int32_t*, int, int, int32_t*, cudaStream_t);
int gather_rows(const void*, const int32_t*, int, void*, int64_t, int64_t, int, cudaStream_t);
int silu_mul(const void*, void*, int, int64_t, int64_t, const int32_t*, cudaStream_t, int64_t ld_in = 0, bool gelu = false);
int quantize_fp8(const void*, int, int64_t, void*, float*, int, int64_t, int64_t, cudaStream_t);
int shared_gate_add(const void*, const void*, const void*, const void*, void*, int, int64_t, int64_t, cudaStream_t);
int moe_combine(const void*, const void*, int, const int32_t*, void*, int, int64_t, int, int64_t, int, cudaStream_t);
int act_quant_1x128(const void*, int, int64_t, void*, float*, int64_t, int64_t, cudaStream_t);
int act_prep(const void*, bool, bool, int64_t, const int32_t*, int, void*, float*, int64_t, int, int, cudaStream_t, const int32_t* n_valid = nullptr);
int act_split_fp8(const void*, bool, int64_t, void*, float*, int64_t, int, cudaStream_t);
int quantize_q4_0(const void*, bool, int64_t, void*, void*, int64_t, int64_t, cudaStream_t);
int resadd_rmsnorm(const void*, void*, const void*, void*, const void*, void*, bool, int64_t, int, float, float, cudaStream_t);
int gated_rmsnorm(const void*, const void*, const void*, void*, bool, int, int, float, cudaStream_t);
int act_split_i8(const void*, bool, int64_t, void*, float*, float*, int64_t, int, cudaStream_t);
int resadd_norm_split_fp8(const void*, void*, const void*, void*, bool, float, float, void*, float*, int64_t, int, cudaStream_t);

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Token-tile height of the streaming kernel's grouped mode, from the mean rows per expert.
static inline int grouped_tile(int64_t rows, int E) {
  const int64_t avg = E > 0 ? (rows + E - 1) / E : rows;
  return avg <= 8 ? 8 : (avg <= 16 ? 16 : (avg <= 32 ? 32 : 64));
}
static inline size_t tile_list_bytes(int64_t rows, int E, int tile) {
  return align_up(16 + 8 * (size_t)((rows + tile - 1) / tile + E), 256);
}

// [pre-passed activations M x K fp16] [per-token scales] [partial sums of the balanced decode mode]
static inline size_t ws_prep_bytes(int64_t M, int64_t K) {
  return align_up((size_t)M * (size_t)K * 2, 256) + align_up((size_t)M * 4, 256);
}

// [e4m3 term rows x K] [per-token scales] of the FP8 decode path
static inline size_t ws_direct_bytes(int64_t M, int64_t K) {
  if (M > 64) return 0;
  return align_up((size_t)umma_w8_direct_rows(M, false) * (size_t)K, 256) + align_up((size_t)M * 4, 256) +
         umma_w8_direct_partial_bytes(M);
}

// [int8 term rows x K] [per-token scales] [per-group activation sums] [partial sums] of the INT4 decode path
static inline size_t ws_i8_bytes(int64_t M, int64_t K) {
  if (M > 16) return 0;
  return align_up((size_t)umma_w4_i8_rows(M) * (size_t)K, 256) + align_up((size_t)M * 4, 256) +
         align_up((size_t)(K / 128) * 16 * 4, 256) + umma_w4_i8_partial_bytes();
}

template <class Args>
static void give_balanced_scratch(Args& ua, void* workspace, int64_t M, int64_t K) {
  if (M > 64) return;
  ua.sk_ws = reinterpret_cast<uint8_t*>(workspace) + ws_prep_bytes(M, K);
  ua.sk_ws_bytes = umma_balanced_ws_bytes(M);
}

}  // namespace b2q

using namespace b2q;

extern "C" {

const char* b2q_strerror(int code) {
  switch (code) {
    case B2Q_OK: return "ok";
    case B2Q_ERR_NULL: return "b2q: a required pointer is NULL";
    case B2Q_ERR_SHAPE: return "b2q: a dimension violates the op's contract";
    case B2Q_ERR_DTYPE: return "b2q: unsupported element type";
    case B2Q_ERR_ALIGN: return "b2q: pointer or row pitch is not 16-byte aligned";
    case B2Q_ERR_LAYOUT: return "b2q: unsupported weight layout";
    case B2Q_ERR_UNSUPPORTED: return "b2q: no kernel for this combination";
    case B2Q_ERR_CUDA: return "b2q: CUDA call failed";
    case B2Q_ERR_WORKSPACE: return "b2q: workspace too small";
    case B2Q_ERR_TIMEOUT: return "b2q: bounded device-side wait expired";
    case B2Q_ERR_LIMIT: return "b2q: size exceeds a built-in capacity";
    default: return "b2q: unknown error code";
  }
}

int b2q_version(void) { return 100; }

int b2q_device_ok(void) {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return B2Q_ERR_CUDA;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return B2Q_ERR_CUDA;
  return major == 10 ? B2Q_OK : B2Q_ERR_UNSUPPORTED;
}

int b2q_quantize_q4_0(const void* x, int act_dtype, int64_t ldx, void* qweight, void* scale_f16, int64_t M, int64_t K,
                      void* stream) {
  if (!x || !qweight || !scale_f16) return B2Q_ERR_NULL;
  if (!is16(act_dtype)) return B2Q_ERR_DTYPE;
  if (M < 0 || K <= 0 || (K % 128) != 0 || ldx < K) return B2Q_ERR_SHAPE;
  if (M > INT32_MAX || K > INT32_MAX) return B2Q_ERR_LIMIT;
  if ((reinterpret_cast<uintptr_t>(x) & 7u) || ((ldx * 2) & 7u)) return B2Q_ERR_ALIGN;
  return quantize_q4_0(x, act_dtype == B2Q_BF16, ldx, qweight, scale_f16, M, K, (cudaStream_t)stream);
}

int b2q_quantize_fp8(const void* w, int w_dtype, int64_t ldw, void* wq, float* scale, int scale_mode, int64_t N, int64_t K,
                     void* stream) {
  if (!w || !wq || !scale) return B2Q_ERR_NULL;
  if (w_dtype != B2Q_BF16 && w_dtype != B2Q_F16 && w_dtype != B2Q_F32) return B2Q_ERR_DTYPE;
  if (scale_mode < 0 || scale_mode > 2) return B2Q_ERR_LAYOUT;
  if (N < 0 || K < 0 || ldw < K) return B2Q_ERR_SHAPE;
  if (N > INT32_MAX || K > INT32_MAX) return B2Q_ERR_LIMIT;
  return quantize_fp8(w, w_dtype, ldw, wq, scale, scale_mode, N, K, (cudaStream_t)stream);
}

int b2q_resadd_rmsnorm(const void* hidden, void* residual, const void* norm_weight, void* normed_out, int act_dtype, int64_t M,
                       int64_t K, float eps, void* stream) {
  if (!hidden || !residual || !norm_weight || !normed_out) return B2Q_ERR_NULL;
  if (!is16(act_dtype)) return B2Q_ERR_DTYPE;
  if (M < 0 || K <= 0 || (K % 8) != 0) return B2Q_ERR_SHAPE;
  if (M > INT32_MAX || K > INT32_MAX) return B2Q_ERR_LIMIT;
  if (!aligned16(hidden) || !aligned16(residual) || !aligned16(norm_weight) || !aligned16(normed_out)) return B2Q_ERR_ALIGN;
  return resadd_rmsnorm(hidden, residual, norm_weight, normed_out, nullptr, nullptr, act_dtype == B2Q_BF16, M, (int)K, eps,
                        1.0f, (cudaStream_t)stream);
}

int b2q_rmsnorm_fused(const void* hidden, void* residual, float scalar, const void* w1, void* out1, const void* w2,
                      void* out2, int act_dtype, int64_t M, int64_t K, float eps, void* stream) {
  if (!residual || !w1 || !out1 || ((w2 == nullptr) != (out2 == nullptr))) return B2Q_ERR_NULL;
  if (!is16(act_dtype)) return B2Q_ERR_DTYPE;
  if (M < 0 || K <= 0 || (K % 8) != 0) return B2Q_ERR_SHAPE;
  if (M > INT32_MAX || K > INT32_MAX) return B2Q_ERR_LIMIT;
  if (!aligned16(residual) || !aligned16(w1) || !aligned16(out1) || (hidden && !aligned16(hidden)) ||
      (w2 && (!aligned16(w2) || !aligned16(out2))))
    return B2Q_ERR_ALIGN;
  return resadd_rmsnorm(hidden, residual, w1, out1, w2, out2, act_dtype == B2Q_BF16, M, (int)K, eps, scalar,
                        (cudaStream_t)stream);
}

int b2q_gated_rmsnorm(const void* x, const void* z, const void* norm_weight, void* out, int act_dtype, int64_t rows, int64_t V,
                      float eps, void* stream) {
  if (!x || !z || !norm_weight || !out) return B2Q_ERR_NULL;
  if (!is16(act_dtype)) return B2Q_ERR_DTYPE;
  if (rows < 0 || V <= 0) return B2Q_ERR_SHAPE;
  if (rows > INT32_MAX || V > INT32_MAX) return B2Q_ERR_LIMIT;
  return gated_rmsnorm(x, z, norm_weight, out, act_dtype == B2Q_BF16, (int)rows, (int)V, eps, (cudaStream_t)stream);
}

void b2q_set_force_kernel(int which) { tls().force_kernel = which; }
void b2q_set_overlap_mode(int mode) { tls().overlap_mode = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }
const char* b2q_last_kernel(void) { return tls().last_kernel; }
uint64_t b2q_launch_count(void) { return tls().launches; }

int b2q_dequant_int4(const void* w, int w_layout, const void* scale, int scale_dtype, void* out, int out_dtype,
                     int64_t N, int64_t K, int group, void* stream) {
  if (!w || !scale || !out) return B2Q_ERR_NULL;
  if (w_layout < 0 || w_layout > 3) return B2Q_ERR_LAYOUT;
  if (!is16(scale_dtype) && scale_dtype != B2Q_F32) return B2Q_ERR_DTYPE;
  if (out_dtype < 0 || out_dtype > 2) return B2Q_ERR_DTYPE;
  if (N < 0 || K < 0 || group <= 0 || (K % group) != 0 || (K % 8) != 0 || (group % 8) != 0) return B2Q_ERR_SHAPE;
  if (!aligned16(out) || !aligned16(w)) return B2Q_ERR_ALIGN;
  if (N == 0 || K == 0) return B2Q_OK;
  return dequant_int4(w, w_layout, scale, scale_dtype, out, out_dtype, N, K, group, (cudaStream_t)stream);
}

int b2q_dequant_fp8(const void* w, int fp8_format, const void* scale, int scale_dtype, int scale_mode, void* out,
                    int out_dtype, int64_t N, int64_t K, void* stream) {
  if (!w || !scale || !out) return B2Q_ERR_NULL;
  if (fp8_format != B2Q_E4M3 && fp8_format != B2Q_E5M2) return B2Q_ERR_DTYPE;
  if (scale_mode < 0 || scale_mode > 2) return B2Q_ERR_LAYOUT;
  if (scale_dtype < 0 || scale_dtype > 2 || out_dtype < 0 || out_dtype > 2) return B2Q_ERR_DTYPE;
  if (N < 0 || K < 0 || (K % 8) != 0) return B2Q_ERR_SHAPE;
  if (!aligned16(out) || (reinterpret_cast<uintptr_t>(w) & 7u)) return B2Q_ERR_ALIGN;
  if (N == 0 || K == 0) return B2Q_OK;
  return dequant_fp8(w, fp8_format, scale, scale_dtype, scale_mode, out, out_dtype, N, K, (cudaStream_t)stream);
}

}  // extern "C"

// peer != nullptr: the output tile is delivered to the reduction slots of its owner ranks instead of to `out`
// (tcgen05 decode kernel only; B2Q_ERR_UNSUPPORTED, with nothing launched, when another kernel would be chosen).
static int linear_int4_core(const void* x, int act_dtype, int64_t ldx, const void* w, int w_layout, const void* scale,
                            int scale_dtype, int64_t s_stride_n, int64_t s_stride_g, void* out, int64_t ldo, int64_t M,
                            int64_t N, int64_t K, int group, void* workspace, size_t workspace_bytes, void* stream,
                            const PeerEpilogue* peer) {
  if (!x || !w || !scale || !out) return B2Q_ERR_NULL;
  if (!is16(act_dtype)) return B2Q_ERR_DTYPE;
  if (scale_dtype < 0 || scale_dtype > 2) return B2Q_ERR_DTYPE;
  if (w_layout < 0 || w_layout > 3) return B2Q_ERR_LAYOUT;
  if (group != 128) return B2Q_ERR_SHAPE;
  if (M < 0 || N < 0 || K <= 0 || (K % group) != 0 || ldx < K || ldo < N) return B2Q_ERR_SHAPE;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return B2Q_ERR_LIMIT;
  if (!aligned16(x) || !aligned16(w) || ((ldx * 2) & 15)) return B2Q_ERR_ALIGN;
  if (M == 0 || N == 0) return B2Q_OK;
  const bool kmajor = (w_layout == B2Q_W4_KMAJOR || w_layout == B2Q_W4_KMAJOR_MARLIN);
  cudaStream_t st = (cudaStream_t)stream;
  const int force = tls().force_kernel;

  UmmaW4Args ua{};
  ua.x = x; ua.ldx = ldx; ua.bf16 = (act_dtype == B2Q_BF16);
  ua.w = w; ua.layout = w_layout; ua.scale = scale; ua.scale_dtype = scale_dtype;
  ua.s_stride_n = s_stride_n; ua.s_stride_g = s_stride_g;
  ua.out = out; ua.ldo = ldo; ua.M = (int)M; ua.N = (int)N; ua.K = (int)K;
  const bool umma_ok = umma_w4_supported(ua);
  if (peer) {
    const bool tiny_p = M <= 32 && N * K <= (int64_t)1 << 25;
    const bool umma_p = force >= 2 || (force == 0 && (kmajor || (M > 8 && !tiny_p)));
    if (!umma_ok || !umma_p || M > 64 || (N % 128) != 0 || force == 5 || (force == 0 && umma_w4_i8_preferred(M, N, K) && M <= 16))
      return B2Q_ERR_UNSUPPORTED;
    ua.peer = peer;
  }
  // the int8 tensor-core path (umma_w4_i8.cu): decode shapes, N-major nibbles, scratch available; on request, or
  // where it measured fastest
  if (!peer && (force == 5 || (force == 0 && umma_w4_i8_preferred(M, N, K))) && umma_ok && !kmajor && M <= 16 && workspace && aligned16(workspace) &&
      workspace_bytes >= b2q_linear_workspace_bytes(M, N, K)) {
    uint8_t* wsb = reinterpret_cast<uint8_t*>(workspace);
    float* inv = reinterpret_cast<float*>(wsb + align_up((size_t)umma_w4_i8_rows(M) * (size_t)K, 256));
    float* xsum = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(inv) + align_up((size_t)M * 4, 256));
    int rc = act_split_i8(x, act_dtype == B2Q_BF16, ldx, workspace, inv, xsum, M, (int)K, st);
    if (rc) return rc;
    UmmaW4I8Args ia{};
    ia.xq = workspace; ia.inv_scale = inv; ia.xsum = xsum;
    ia.w = w; ia.xor_mask = (w_layout == B2Q_W4_NMAJOR_S4) ? 0x88888888u : 0u;
    ia.scale = scale; ia.scale_dtype = scale_dtype; ia.s_stride_n = s_stride_n; ia.s_stride_g = s_stride_g;
    ia.out = out; ia.ldo = ldo; ia.out_bf16 = act_dtype == B2Q_BF16; ia.M = (int)M; ia.N = (int)N; ia.K = (int)K;
    ia.partials = reinterpret_cast<uint8_t*>(xsum) + align_up((size_t)(K / 128) * 16 * 4, 256);
    ia.partial_bytes = umma_w4_i8_partial_bytes();
    return umma_w4_i8_linear(ia, st);
  }
  // measured on B200: the mma.sync streaming kernel wins only for a handful of tokens (its per-token cost is
  // fragment traffic), the tcgen05 kernel is flat in M up to 64 and the only one for K-major layouts and prefill
  // small weights at small M: one launch of the streaming kernel beats pre-pass + GEMM
  const bool tiny = M <= 32 && N * K <= (int64_t)1 << 25;
  const bool want_umma = force >= 2 || (force == 0 && (kmajor || (M > 8 && !tiny)));
  if (umma_ok && want_umma) {
    // With scratch, activations go through the pre-pass (fp16, per-token power-of-two scale, pair order of
    // the magic-number transform) and the transform's integer work drops from 12 to 5 operations per word.
    const bool prep = workspace && aligned16(workspace) && workspace_bytes >= b2q_linear_workspace_bytes(M, N, K) &&
                      force != 3;
    ua.out_bf16 = ua.bf16;
    if (prep) {
      float* inv = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + align_up((size_t)M * (size_t)K * 2, 256));
      const int perm = w_layout == B2Q_W4_KMAJOR_MARLIN ? 2 : 1;
      int rc = act_prep(x, act_dtype == B2Q_BF16, false, ldx, nullptr, 1, workspace, inv, M, (int)K, perm, st);
      if (rc) return rc;
      ua.x = workspace; ua.ldx = K; ua.bf16 = false; ua.tok_scale = inv; ua.magic = true; ua.after_prep = true;
      give_balanced_scratch(ua, workspace, M, K);
    }
    return umma_w4_linear(ua, st);
  }
  if (kmajor) return B2Q_ERR_UNSUPPORTED;

  SmallMParams p{};
  p.x = x; p.ldx = ldx;
  p.w = reinterpret_cast<const uint8_t*>(w); p.w_row_bytes = K / 2;
  p.scale = scale; p.scale_dtype = scale_dtype; p.s_stride_n = s_stride_n; p.s_stride_g = s_stride_g;
  p.out = out; p.ldo = ldo; p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.xor_mask = (w_layout == B2Q_W4_NMAJOR_S4) ? 0x88888888u : 0u;
  return smallm_int4(p, act_dtype == B2Q_BF16, (int)M, 0, st);
}

extern "C" {

int b2q_allreduce_sum(void* comm, const void* in, int dtype, int64_t ldi, int64_t M, int64_t N, double wait_limit_ms,
                      void** out, void* stream);

int b2q_linear_int4(const void* x, int act_dtype, int64_t ldx, const void* w, int w_layout, const void* scale,
                    int scale_dtype, int64_t s_stride_n, int64_t s_stride_g, void* out, int64_t ldo, int64_t M,
                    int64_t N, int64_t K, int group, void* workspace, size_t workspace_bytes, void* stream) {
  return linear_int4_core(x, act_dtype, ldx, w, w_layout, scale, scale_dtype, s_stride_n, s_stride_g, out, ldo, M, N, K,
                          group, workspace, workspace_bytes, stream, nullptr);
}

int b2q_linear_int4_allreduce(const void* x, int act_dtype, int64_t ldx, const void* w, int w_layout, const void* scale,
                              int scale_dtype, int64_t s_stride_n, int64_t s_stride_g, void* partial, int64_t ldp,
                              int64_t M, int64_t N, int64_t K, int group, void* workspace, size_t workspace_bytes,
                              void* comm, double wait_limit_ms, void** out, void* stream) {
  if (!comm || !out || !partial) return B2Q_ERR_NULL;
  PeerEpilogue pe;
  int rc = peer_epilogue(comm, M, N, &pe);
  if (rc == B2Q_OK) {
    rc = linear_int4_core(x, act_dtype, ldx, w, w_layout, scale, scale_dtype, s_stride_n, s_stride_g, partial, ldp, M, N, K,
                          group, workspace, workspace_bytes, stream, &pe);
    if (rc == B2Q_OK) return b2q_allreduce_sum(comm, nullptr, act_dtype, 0, M, N, wait_limit_ms, out, stream);
  }
  if (rc != B2Q_ERR_UNSUPPORTED && rc != B2Q_ERR_SHAPE) return rc;
  // another kernel serves this shape: GEMM into `partial`, then the reduction delivers the tile itself
  rc = linear_int4_core(x, act_dtype, ldx, w, w_layout, scale, scale_dtype, s_stride_n, s_stride_g, partial, ldp, M, N, K,
                        group, workspace, workspace_bytes, stream, nullptr);
  if (rc) return rc;
  return b2q_allreduce_sum(comm, partial, act_dtype, ldp, M, N, wait_limit_ms, out, stream);
}

size_t b2q_linear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  (void)N;
  const size_t a = ws_prep_bytes(M, K) + umma_balanced_ws_bytes(M), b = ws_i8_bytes(M, K);
  return a > b ? a : b;
}
size_t b2q_linear_fp8_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const size_t a = b2q_linear_workspace_bytes(M, N, K), b = ws_direct_bytes(M, K);
  return a > b ? a : b;
}

}  // extern "C"

// Residual add + RMSNorm in front of the GEMV: when `nf` is given, x is the normed_out buffer the front end fills.
struct NormFront { const void* hidden; void* residual; const void* norm_weight; float eps, scalar; };

static int linear_fp8_core(const void* x, int act_dtype, int64_t ldx, const void* w, int fp8_format, const void* scale,
                           int scale_dtype, int scale_mode, void* out, int64_t ldo, int64_t M, int64_t N, int64_t K,
                           void* workspace, size_t workspace_bytes, void* stream, const NormFront* nf) {
  if (!x || !w || !scale || !out) return B2Q_ERR_NULL;
  if (!is16(act_dtype)) return B2Q_ERR_DTYPE;
  if (fp8_format != B2Q_E4M3 && fp8_format != B2Q_E5M2) return B2Q_ERR_DTYPE;
  if (scale_mode < 0 || scale_mode > 2) return B2Q_ERR_LAYOUT;
  if (scale_dtype < 0 || scale_dtype > 2) return B2Q_ERR_DTYPE;
  if (scale_mode == B2Q_SCALE_BLOCK128 && (scale_dtype != B2Q_F32 || fp8_format != B2Q_E4M3)) return B2Q_ERR_DTYPE;
  if (M < 0 || N < 0 || K <= 0 || (K % 16) != 0 || ldx < K || ldo < N) return B2Q_ERR_SHAPE;
  if (scale_mode == B2Q_SCALE_BLOCK128 && (K % 128) != 0) return B2Q_ERR_SHAPE;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return B2Q_ERR_LIMIT;
  if (!aligned16(x) || !aligned16(w) || ((ldx * 2) & 15)) return B2Q_ERR_ALIGN;
  if (M == 0 || N == 0) return B2Q_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int force = tls().force_kernel;

  UmmaW8Args ua{};
  ua.x = x; ua.ldx = ldx; ua.bf16 = (act_dtype == B2Q_BF16); ua.out_bf16 = ua.bf16; ua.tok_scale = nullptr;
  ua.w = w; ua.fmt = fp8_format; ua.scale = scale; ua.scale_dtype = scale_dtype; ua.scale_mode = scale_mode;
  ua.out = out; ua.ldo = ldo; ua.M = (int)M; ua.N = (int)N; ua.K = (int)K;
  const bool umma_ok = umma_w8_supported(ua);
  // bf16 activations + scratch: convert them once to per-token-scaled fp16 so the weight decode is one cvt per pair
  const bool have_ws = workspace && aligned16(workspace) && workspace_bytes >= b2q_linear_fp8_workspace_bytes(M, N, K) &&
                       force != 3;
  // decode shapes with one scale per row or per tensor: weights stay e4m3 all the way into the 8-bit MMA, the
  // activations are split into e4m3 terms instead (exact), see umma_w8_direct.cu
  if (force == 0 && have_ws && M <= 64 && scale_mode != B2Q_SCALE_BLOCK128 && umma_ok) {
    float* inv = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) +
                                          align_up((size_t)umma_w8_direct_rows(M, false) * (size_t)K, 256));
    // with a norm front end, ONE pre-pass launch does residual add, RMSNorm (normed_out = x) and the term split
    int rc = nf ? resadd_norm_split_fp8(nf->hidden, nf->residual, nf->norm_weight, const_cast<void*>(x), act_dtype == B2Q_BF16,
                                        nf->eps, nf->scalar, workspace, inv, M, (int)K, st)
                : act_split_fp8(x, act_dtype == B2Q_BF16, ldx, workspace, inv, M, (int)K, st);
    if (rc) return rc;
    UmmaW8DirectArgs da{};
    da.xq = workspace; da.inv_scale = inv; da.terms = act_dtype == B2Q_BF16 ? 2 : 3;
    da.w = w; da.fmt = fp8_format; da.scale = scale; da.scale_dtype = scale_dtype; da.scale_mode = scale_mode;
    da.out = out; da.ldo = ldo; da.out_bf16 = act_dtype == B2Q_BF16; da.M = (int)M; da.N = (int)N; da.K = (int)K;
    da.partials = reinterpret_cast<uint8_t*>(inv) + align_up((size_t)M * 4, 256);
    da.partial_bytes = umma_w8_direct_partial_bytes(M);
    return umma_w8_direct_linear(da, st);
  }
  if (nf) {      // every other kernel family: the norm as its own launch, then the ordinary path on normed_out
    int rc = resadd_rmsnorm(nf->hidden, nf->residual, nf->norm_weight, const_cast<void*>(x), nullptr, nullptr,
                            act_dtype == B2Q_BF16, M, (int)K, nf->eps, nf->scalar, st);
    if (rc) return rc;
  }
  const bool prep = act_dtype == B2Q_BF16 && have_ws && (K % 8) == 0;
  const bool want_umma = force >= 2 || (force == 0 && (M > 4 || prep || act_dtype == B2Q_F16));
  if (umma_ok && want_umma) {
    if (prep) {
      float* inv = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + align_up((size_t)M * (size_t)K * 2, 256));
      int rc = act_prep(x, true, false, ldx, nullptr, 1, workspace, inv, M, (int)K, 0, st);
      if (rc) return rc;
      ua.x = workspace; ua.ldx = K; ua.bf16 = false; ua.out_bf16 = true; ua.tok_scale = inv; ua.after_prep = true;
    }
    if (have_ws) give_balanced_scratch(ua, workspace, M, K);
    return umma_w8_linear(ua, st);
  }

  SmallMParams p{};
  p.x = x; p.ldx = ldx;
  p.w = reinterpret_cast<const uint8_t*>(w); p.w_row_bytes = K;
  p.scale = scale; p.scale_dtype = scale_dtype;
  p.s_stride_n = (scale_mode == B2Q_SCALE_CHANNEL) ? 1 : 0;
  p.out = out; p.ldo = ldo; p.M = (int)M; p.N = (int)N; p.K = (int)K;
  const int smode = scale_mode == B2Q_SCALE_BLOCK128 ? SM_BLOCK : SM_POST;
  return act_dtype == B2Q_BF16 ? smallm_fp8_bf16(p, fp8_format, smode, (int)M, 0, st)
                               : smallm_fp8_f16(p, fp8_format, smode, (int)M, 0, st);
}

extern "C" {

int b2q_linear_fp8(const void* x, int act_dtype, int64_t ldx, const void* w, int fp8_format, const void* scale,
                   int scale_dtype, int scale_mode, void* out, int64_t ldo, int64_t M, int64_t N, int64_t K,
                   void* workspace, size_t workspace_bytes, void* stream) {
  return linear_fp8_core(x, act_dtype, ldx, w, fp8_format, scale, scale_dtype, scale_mode, out, ldo, M, N, K, workspace,
                         workspace_bytes, stream, nullptr);
}

int b2q_resadd_norm_linear_fp8(const void* hidden, void* residual, const void* norm_weight, void* normed_out, float eps,
                               float scalar, int act_dtype, const void* w, int fp8_format, const void* scale, int scale_dtype,
                               int scale_mode, void* out, int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace,
                               size_t workspace_bytes, void* stream) {
  if (!hidden || !residual || !norm_weight || !normed_out) return B2Q_ERR_NULL;
  if (!is16(act_dtype)) return B2Q_ERR_DTYPE;
  if (K <= 0 || (K % 16) != 0) return B2Q_ERR_SHAPE;
  if (!aligned16(hidden) || !aligned16(residual) || !aligned16(norm_weight) || !aligned16(normed_out)) return B2Q_ERR_ALIGN;
  const NormFront nf{hidden, residual, norm_weight, eps, scalar};
  return linear_fp8_core(normed_out, act_dtype, K, w, fp8_format, scale, scale_dtype, scale_mode, out, ldo, M, N, K, workspace,
                         workspace_bytes, stream, &nf);
}

int b2q_act_quant_fp8_1x128(const void* x, int act_dtype, int64_t ldx, void* xq, float* xs, int64_t M, int64_t K,
                            void* stream) {
  if (!x || !xq || !xs) return B2Q_ERR_NULL;
  if (!is16(act_dtype)) return B2Q_ERR_DTYPE;
  if (M < 0 || K < 0 || (K % 128) != 0 || ldx < K) return B2Q_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) & 7u) || ((ldx * 2) & 7) || (reinterpret_cast<uintptr_t>(xq) & 3u)) return B2Q_ERR_ALIGN;
  return act_quant_1x128(x, act_dtype, ldx, xq, xs, M, K, (cudaStream_t)stream);
}

int b2q_gemm_fp8_block_w8a8(const void* xq, const float* xs, const void* w, const float* ws, void* out, int out_dtype,
                            int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream) {
  if (!xq || !xs || !w || !ws || !out) return B2Q_ERR_NULL;
  if (!is16(out_dtype)) return B2Q_ERR_DTYPE;
  if (M < 0 || N < 0 || K <= 0 || (K % 128) != 0 || ldo < N) return B2Q_ERR_SHAPE;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return B2Q_ERR_LIMIT;
  if (!aligned16(xq) || !aligned16(w)) return B2Q_ERR_ALIGN;
  if (M == 0 || N == 0) return B2Q_OK;
  UmmaW8A8Args a{};
  a.xq = xq; a.xs = xs; a.w = w; a.ws = ws; a.out = out; a.bf16 = (out_dtype == B2Q_BF16); a.ldo = ldo;
  a.M = (int)M; a.N = (int)N; a.K = (int)K;
  return umma_w8a8_block(a, (cudaStream_t)stream);
}

int b2q_moe_topk(const void* logits, int logits_dtype, int64_t T, int E, int top_k, int renorm, void* weights,
                 int w_dtype, int32_t* ids, void* stream) {
  if (!logits || !weights || !ids) return B2Q_ERR_NULL;
  if (logits_dtype < 0 || logits_dtype > 2 || w_dtype < 0 || w_dtype > 2) return B2Q_ERR_DTYPE;
  if (T < 0 || E <= 0 || top_k <= 0 || top_k > E) return B2Q_ERR_SHAPE;
  if (E > 1024 || top_k > 32) return B2Q_ERR_LIMIT;
  return moe_topk(logits, logits_dtype, T, E, top_k, renorm, weights, w_dtype, ids, (cudaStream_t)stream);
}

size_t b2q_moe_route_workspace_bytes(int64_t n_pairs, int E) { return moe_route_workspace_bytes(n_pairs, E); }

int b2q_moe_route(const int32_t* ids, int64_t n_pairs, int E, int32_t* expert_offsets, int32_t* expert_tokens,
                  int32_t* pair_to_perm, int32_t* rows_per_expert, void* workspace, size_t workspace_bytes,
                  void* stream) {
  if (!ids || !expert_offsets || !expert_tokens || !workspace) return B2Q_ERR_NULL;
  if (n_pairs < 0 || E <= 0) return B2Q_ERR_SHAPE;
  if (E > 1024 || n_pairs > INT32_MAX) return B2Q_ERR_LIMIT;
  if (workspace_bytes < moe_route_workspace_bytes(n_pairs, E)) return B2Q_ERR_WORKSPACE;
  return moe_route(ids, n_pairs, E, expert_offsets, expert_tokens, pair_to_perm, rows_per_expert, workspace,
                   (cudaStream_t)stream);
}

int b2q_gather_rows(const void* src, const int32_t* idx, int div, void* dst, int64_t rows, int64_t cols,
                    int elem_bytes, void* stream) {
  if (!src || !dst) return B2Q_ERR_NULL;
  if (rows < 0 || cols < 0 || div <= 0 || elem_bytes <= 0 || ((cols * elem_bytes) % 16) != 0) return B2Q_ERR_SHAPE;
  if (!aligned16(src) || !aligned16(dst)) return B2Q_ERR_ALIGN;
  return gather_rows(src, idx, div, dst, rows, cols, elem_bytes, (cudaStream_t)stream);
}

int b2q_silu_mul(const void* in, void* out, int dtype, int64_t rows, int64_t I, void* stream) {
  if (!in || !out) return B2Q_ERR_NULL;
  if (!is16(dtype)) return B2Q_ERR_DTYPE;
  if (rows < 0 || I < 0 || (I % 8) != 0) return B2Q_ERR_SHAPE;
  if (!aligned16(in) || !aligned16(out)) return B2Q_ERR_ALIGN;
  return silu_mul(in, out, dtype, rows, I, nullptr, (cudaStream_t)stream);
}

int b2q_gelu_tanh_mul(const void* in, void* out, int dtype, int64_t rows, int64_t I, void* stream) {
  if (!in || !out) return B2Q_ERR_NULL;
  if (!is16(dtype)) return B2Q_ERR_DTYPE;
  if (rows < 0 || I < 0 || (I % 8) != 0) return B2Q_ERR_SHAPE;
  if (!aligned16(in) || !aligned16(out)) return B2Q_ERR_ALIGN;
  return silu_mul(in, out, dtype, rows, I, nullptr, (cudaStream_t)stream, 0, true);
}

int b2q_moe_combine(const void* y, const void* w, int w_dtype, const int32_t* perm, void* out, int dtype, int64_t T,
                    int top_k, int64_t H, int w_by_row, void* stream) {
  if (!y || !out) return B2Q_ERR_NULL;
  if (!is16(dtype) || w_dtype < 0 || w_dtype > 2) return B2Q_ERR_DTYPE;
  if (T < 0 || top_k <= 0 || H < 0 || (H % 8) != 0) return B2Q_ERR_SHAPE;
  if (!aligned16(y) || !aligned16(out)) return B2Q_ERR_ALIGN;
  return moe_combine(y, w, w_dtype, perm, out, dtype, T, top_k, H, w_by_row, (cudaStream_t)stream);
}

int b2q_moe_shared_gate_add(const void* x, const void* gate_w, const void* shared, const void* routed, void* out,
                            int dtype, int64_t T, int64_t H, void* stream) {
  if (!x || !gate_w || !shared || !routed || !out) return B2Q_ERR_NULL;
  if (!is16(dtype)) return B2Q_ERR_DTYPE;
  if (T < 0 || H <= 0 || (H % 8) != 0 || T > INT32_MAX) return B2Q_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(gate_w) || !aligned16(shared) || !aligned16(routed) || !aligned16(out)) return B2Q_ERR_ALIGN;
  return shared_gate_add(x, gate_w, shared, routed, out, dtype, T, H, (cudaStream_t)stream);
}

size_t b2q_moe_gemm_workspace_bytes(int64_t rows, int E, int64_t N, int64_t K, int act, int gather) {
  // [tile list for the smallest (8-row) tiling] [gathered activations rows x K] [un-activated rows x N]
  // [tile list] [pre-passed activations rows x K fp16] [per-row scales] [un-activated rows x N]
  (void)gather;
  size_t b = tile_list_bytes(rows, E, 8);
  b += align_up((size_t)rows * (size_t)K * 2, 256) + align_up((size_t)rows * 4, 256);
  if (act == B2Q_ACT_SILU_MUL || act == B2Q_ACT_GELU_TANH_MUL) b += align_up((size_t)rows * (size_t)N * 2, 256);
  return b;
}

int b2q_device_status(int* out) {
  if (!out) return B2Q_ERR_NULL;
  return umma_read_status(out);
}

int b2q_device_status_reset(void) { return umma_reset_status(); }

int b2q_selftest_bounded_wait(int code, int* gave_up, void* stream) {
  if (!gave_up) return B2Q_ERR_NULL;
  if (code <= 0) return B2Q_ERR_SHAPE;
  return umma_selftest_bounded_wait(code, gave_up, (cudaStream_t)stream);
}

// Shared tail of the grouped GEMMs once the kernel family is chosen: optional row gather in
// front of the tcgen05 kernel, optional SiLU*mul behind either kernel.
struct GroupedPlan {
  uint8_t* tiles; uint8_t* xg; float* inv; uint8_t* g;
};
static GroupedPlan plan_workspace(void* ws, int64_t rows, int E, int64_t K, bool) {
  GroupedPlan pl;
  pl.tiles = reinterpret_cast<uint8_t*>(ws);
  pl.xg = pl.tiles + tile_list_bytes(rows, E, 8);
  pl.inv = reinterpret_cast<float*>(pl.xg + align_up((size_t)rows * (size_t)K * 2, 256));
  pl.g = reinterpret_cast<uint8_t*>(pl.inv) + align_up((size_t)rows * 4, 256);
  return pl;
}

int b2q_moe_gemm_int4(const void* x, int act_dtype, int64_t ldx, const int32_t* row_map, int row_div, const void* w,
                      int w_layout, const void* scale, int scale_dtype, const int32_t* expert_offsets, int E,
                      void* out, int64_t ldo, const int32_t* out_map, int64_t rows, int64_t N, int64_t K, int group,
                      int act, void* workspace, size_t workspace_bytes, void* stream) {
  if (!x || !w || !scale || !expert_offsets || !out || !workspace) return B2Q_ERR_NULL;
  if (!is16(act_dtype) || scale_dtype < 0 || scale_dtype > 2) return B2Q_ERR_DTYPE;
  if (w_layout < 0 || w_layout > 3) return B2Q_ERR_LAYOUT;
  if (group != 128) return B2Q_ERR_SHAPE;
  const bool gated_in = act == B2Q_ACT_SILU_MUL_IN;
  if (rows < 0 || N <= 0 || K <= 0 || (K % group) != 0 || E <= 0 || ldx < (gated_in ? 2 * K : K)) return B2Q_ERR_SHAPE;
  if (act != B2Q_ACT_NONE && act != B2Q_ACT_SILU_MUL && !gated_in) return B2Q_ERR_UNSUPPORTED;
  if (gated_in && row_map) return B2Q_ERR_UNSUPPORTED;
  if (act == B2Q_ACT_SILU_MUL && ((N % 16) != 0 || ldo != N / 2)) return B2Q_ERR_SHAPE;
  if (act != B2Q_ACT_SILU_MUL && ldo < N) return B2Q_ERR_SHAPE;
  if (E > 1024 || rows > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return B2Q_ERR_LIMIT;
  if (row_map && row_div <= 0) return B2Q_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(w) || !aligned16(workspace) || ((ldx * 2) & 15)) return B2Q_ERR_ALIGN;
  if (workspace_bytes < b2q_moe_gemm_workspace_bytes(rows, E, N, K, act, row_map != nullptr)) return B2Q_ERR_WORKSPACE;
  if (rows == 0) return B2Q_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool kmajor = (w_layout == B2Q_W4_KMAJOR || w_layout == B2Q_W4_KMAJOR_MARLIN);
  const bool bf = act_dtype == B2Q_BF16;
  const int force = tls().force_kernel;
  const GroupedPlan pl = plan_workspace(workspace, rows, E, K, row_map != nullptr);
  int32_t* tiles = reinterpret_cast<int32_t*>(pl.tiles);
  const bool act_out = act == B2Q_ACT_SILU_MUL;
  void* gemm_out = act_out ? pl.g : out;
  const int64_t gemm_ldo = act_out ? N : ldo;
  const int32_t* gemm_out_map = act_out ? nullptr : out_map;
  int rc;

  UmmaW4Args ua{};
  ua.x = x; ua.ldx = ldx; ua.bf16 = bf;
  ua.w = w; ua.layout = w_layout; ua.scale = scale; ua.scale_dtype = scale_dtype;
  ua.s_stride_n = kmajor ? 1 : K / group; ua.s_stride_g = kmajor ? N : 1;
  ua.out = gemm_out; ua.ldo = gemm_ldo; ua.M = (int)rows; ua.N = (int)N; ua.K = (int)K;
  ua.expert_offsets = expert_offsets; ua.E = E; ua.out_map = gemm_out_map; ua.tiles = tiles;
  const int64_t avg = (rows + E - 1) / E;
  // measured on 128 experts of [1536 x 2048] / [2048 x 768] at 1 to 256 tokens (top-8): the tcgen05 kernel behind its
  // pre-pass beats the streaming kernel at every batch (49 / 76 / 139 / 205 / 284 us per pipeline pass against
  // 60 / 94 / 177 / 286 / 467), so only experts too small to matter stay on the streaming kernel
  const bool want_umma = force == 2 || (force == 0 && (kmajor || avg > 16 || N * K >= ((int64_t)1 << 20)));
  ua.out_bf16 = bf;
  if (umma_w4_supported(ua) && want_umma) {
    // gather (if any), fp16 re-scaling and pair permutation in one pre-pass over the rows
    // (with a gated input also silu(gate) * up, so that the gate_up result is read once and never re-written)
    // `rows` may be an upper bound (expert-parallel receive buffers of fixed capacity): the rows actually routed
    // to these experts are expert_offsets[E], known on the device only
    rc = act_prep(x, bf, gated_in, ldx, row_map, row_div, pl.xg, pl.inv, rows, (int)K,
                  w_layout == B2Q_W4_KMAJOR_MARLIN ? 2 : 1, st, expert_offsets + E);
    if (rc) return rc;
    ua.x = pl.xg; ua.ldx = K; ua.bf16 = false; ua.tok_scale = pl.inv; ua.magic = true;
    const int tile = umma_w4_token_tile(ua);
    rc = moe_build_tiles(expert_offsets, E, tile, tiles, st);
    if (rc) return rc;
    ua.tile_cap = (int)((rows + tile - 1) / tile + E);
    rc = umma_w4_linear(ua, st);
  } else {
    if (kmajor) return B2Q_ERR_UNSUPPORTED;
    const void* xin = x;
    int64_t ldin = ldx;
    if (gated_in) {          // few rows per expert: activate into the scratch first, then the plain grouped kernel
      rc = silu_mul(x, pl.xg, act_dtype, rows, K, nullptr, st, ldx);
      if (rc) return rc;
      xin = pl.xg; ldin = K;
    }
    const int tile = grouped_tile(rows, E);
    rc = moe_build_tiles(expert_offsets, E, tile, tiles, st);
    if (rc) return rc;
    SmallMParams p{};
    p.x = xin; p.ldx = ldin;
    p.w = reinterpret_cast<const uint8_t*>(w); p.w_row_bytes = K / 2;
    p.scale = scale; p.scale_dtype = scale_dtype; p.s_stride_n = K / group; p.s_stride_g = 1;
    p.M = (int)rows; p.N = (int)N; p.K = (int)K;
    p.xor_mask = (w_layout == B2Q_W4_NMAJOR_S4) ? 0x88888888u : 0u;
    p.tiles = tiles; p.expert_offsets = expert_offsets; p.row_map = row_map; p.row_div = row_div > 0 ? row_div : 1;
    p.w_expert_bytes = N * (K / 2); p.s_expert_elems = N * (K / group);
    p.out = gemm_out; p.ldo = gemm_ldo; p.out_map = gemm_out_map;
    rc = smallm_int4(p, bf, tile, (int)((rows + tile - 1) / tile + E), st);
  }
  if (rc || !act_out) return rc;
  return silu_mul(pl.g, out, act_dtype, rows, N / 2, out_map, st);
}

int b2q_moe_gemm_fp8(const void* x, int act_dtype, int64_t ldx, const int32_t* row_map, int row_div, const void* w,
                     int fp8_format, const float* scale, int scale_mode, const int32_t* expert_offsets, int E,
                     void* out, int64_t ldo, const int32_t* out_map, int64_t rows, int64_t N, int64_t K, int act,
                     void* workspace, size_t workspace_bytes, void* stream) {
  if (!x || !w || !scale || !expert_offsets || !out || !workspace) return B2Q_ERR_NULL;
  if (!is16(act_dtype)) return B2Q_ERR_DTYPE;
  if (fp8_format != B2Q_E4M3 && fp8_format != B2Q_E5M2) return B2Q_ERR_DTYPE;
  if (scale_mode < 0 || scale_mode > 2) return B2Q_ERR_LAYOUT;
  if (scale_mode == B2Q_SCALE_BLOCK128 && fp8_format != B2Q_E4M3) return B2Q_ERR_DTYPE;
  if (rows < 0 || N <= 0 || K <= 0 || (K % 16) != 0 || E <= 0 || ldx < K) return B2Q_ERR_SHAPE;
  if (scale_mode == B2Q_SCALE_BLOCK128 && ((K % 128) != 0 || (N % 128) != 0)) return B2Q_ERR_SHAPE;
  if (act != B2Q_ACT_NONE && act != B2Q_ACT_SILU_MUL && act != B2Q_ACT_GELU_TANH_MUL) return B2Q_ERR_UNSUPPORTED;
  if (act != B2Q_ACT_NONE && ((N % 16) != 0 || ldo != N / 2)) return B2Q_ERR_SHAPE;
  if (act == B2Q_ACT_NONE && ldo < N) return B2Q_ERR_SHAPE;
  if (E > 1024 || rows > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return B2Q_ERR_LIMIT;
  if (row_map && row_div <= 0) return B2Q_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(w) || !aligned16(workspace) || ((ldx * 2) & 15)) return B2Q_ERR_ALIGN;
  if (workspace_bytes < b2q_moe_gemm_workspace_bytes(rows, E, N, K, act, row_map != nullptr)) return B2Q_ERR_WORKSPACE;
  if (rows == 0) return B2Q_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool bf = act_dtype == B2Q_BF16;
  const int force = tls().force_kernel;
  const GroupedPlan pl = plan_workspace(workspace, rows, E, K, row_map != nullptr);
  int32_t* tiles = reinterpret_cast<int32_t*>(pl.tiles);
  void* gemm_out = act == B2Q_ACT_NONE ? out : pl.g;
  const int64_t gemm_ldo = act == B2Q_ACT_NONE ? ldo : N;
  const int32_t* gemm_out_map = act == B2Q_ACT_NONE ? out_map : nullptr;
  const int64_t kblocks = (K + 127) / 128, nblocks = (N + 127) / 128;
  const int64_t s_expert = scale_mode == B2Q_SCALE_CHANNEL ? N : (scale_mode == B2Q_SCALE_TENSOR ? 1 : nblocks * kblocks);
  int rc;

  UmmaW8Args ua{};
  ua.x = x; ua.ldx = ldx; ua.bf16 = bf;
  ua.w = w; ua.fmt = fp8_format; ua.scale = scale; ua.scale_dtype = B2Q_F32; ua.scale_mode = scale_mode;
  ua.out = gemm_out; ua.ldo = gemm_ldo; ua.M = (int)rows; ua.N = (int)N; ua.K = (int)K;
  ua.expert_offsets = expert_offsets; ua.E = E; ua.out_map = gemm_out_map; ua.tiles = tiles; ua.s_expert_elems = s_expert;
  const int64_t avg = (rows + E - 1) / E;
  const bool want_umma = force == 2 || (force == 0 && avg > 16);
  if (umma_w8_supported(ua) && want_umma) {
    if (row_map) {
      rc = gather_rows(x, row_map, row_div, pl.xg, rows, K, 2, st);
      if (rc) return rc;
      ua.x = pl.xg; ua.ldx = K;
    }
    const int tile = umma_w8_token_tile(ua);
    rc = moe_build_tiles(expert_offsets, E, tile, tiles, st);
    if (rc) return rc;
    ua.tile_cap = (int)((rows + tile - 1) / tile + E);
    rc = umma_w8_linear(ua, st);
  } else {
    const int tile = grouped_tile(rows, E);
    rc = moe_build_tiles(expert_offsets, E, tile, tiles, st);
    if (rc) return rc;
    SmallMParams p{};
    p.x = x; p.ldx = ldx;
    p.w = reinterpret_cast<const uint8_t*>(w); p.w_row_bytes = K;
    p.scale = scale; p.scale_dtype = B2Q_F32; p.s_stride_n = (scale_mode == B2Q_SCALE_CHANNEL) ? 1 : 0;
    p.M = (int)rows; p.N = (int)N; p.K = (int)K;
    p.tiles = tiles; p.expert_offsets = expert_offsets; p.row_map = row_map; p.row_div = row_div > 0 ? row_div : 1;
    p.w_expert_bytes = N * K; p.s_expert_elems = s_expert;
    p.out = gemm_out; p.ldo = gemm_ldo; p.out_map = gemm_out_map;
    const int smode = scale_mode == B2Q_SCALE_BLOCK128 ? SM_BLOCK : SM_POST;
    const int cap = (int)((rows + tile - 1) / tile + E);
    rc = bf ? smallm_fp8_bf16(p, fp8_format, smode, tile, cap, st) : smallm_fp8_f16(p, fp8_format, smode, tile, cap, st);
  }
  if (rc || act == B2Q_ACT_NONE) return rc;
  return silu_mul(pl.g, out, act_dtype, rows, N / 2, out_map, st, 0, act == B2Q_ACT_GELU_TANH_MUL);
}

}  // extern "C"
