/* b2q.h — C ABI of libb2q.so: B200 (sm_100a) quantized-linear hot path.
 *
 * Every entry point takes raw DEVICE pointers and plain integers, launches on the
 * CUDA stream it is given (a cudaStream_t passed as void*; NULL = legacy default
 * stream), never synchronises the host, never allocates, never throws and never
 * aborts.  The return value is 0 on success or a negative B2Q_ERR_* code; a
 * message is available from b2q_strerror().  Nothing is retained past the call.
 *
 * Each group below cites the interface of intel/llm-scaler's
 * vllm/custom-esimd-kernels-vllm package (paths relative to that directory)
 * that it replaces.  The torch custom-op layer in
 * custom_esimd_kernels_vllm/_register.py binds these symbols through ctypes
 * under the reference's own schema strings.
 */
#ifndef B2Q_H_
#define B2Q_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define B2Q_API __attribute__((visibility("default")))
#else
#define B2Q_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define B2Q_OK                 0
#define B2Q_ERR_NULL          -1  /* a required pointer is NULL                     */
#define B2Q_ERR_SHAPE         -2  /* a dimension violates the op's contract         */
#define B2Q_ERR_DTYPE         -3  /* unknown / unsupported element type code        */
#define B2Q_ERR_ALIGN         -4  /* a pointer or pitch is not 16-byte aligned      */
#define B2Q_ERR_LAYOUT        -5  /* unknown / unsupported weight layout code       */
#define B2Q_ERR_UNSUPPORTED   -6  /* valid request with no kernel behind it yet     */
#define B2Q_ERR_CUDA          -7  /* a CUDA runtime / driver call failed            */
#define B2Q_ERR_WORKSPACE     -8  /* caller-provided workspace is too small         */
#define B2Q_ERR_TIMEOUT       -9  /* a bounded device-side wait expired             */
#define B2Q_ERR_LIMIT        -10  /* size exceeds a fixed built-in capacity         */

/* ---- element types of activations / outputs / scales -------------------- */
#define B2Q_BF16 0
#define B2Q_F16  1
#define B2Q_F32  2

/* ---- INT4 weight layouts (value = (q - 8) * scale, q in [0,15]) ---------
 * NMAJOR        int32 [N, K/8] == uint8 [N, K/2]; nibble i of a word (bits
 *               4i..4i+3) is k = 8*word + i ("low nibble = even k").
 *               Scales [N, K/g].              (csrc/xpu/q4_0_quant.sycl:9-13)
 * KMAJOR        int32 [K/8, N] contiguous, same nibble order; scales [K/g, N]
 *               (GPTQ / oneDNN view materialised; tests/test_moe_int4_kernel.py:384-396)
 * KMAJOR_MARLIN int32 [K/8, N] with nibbles shuffled [0,4,1,5,2,6,3,7]; scales
 *               [K/g, N]  (csrc/moe_prefill/moe_prefill_int4.sycl:128-137)
 * NMAJOR_S4     uint8 [N, K/2] two's-complement nibbles (value = s4 * scale)
 *               (csrc/moe_batch/int4_nmajor_gemm.h:137)
 */
#define B2Q_W4_NMAJOR        0
#define B2Q_W4_KMAJOR        1
#define B2Q_W4_KMAJOR_MARLIN 2
#define B2Q_W4_NMAJOR_S4     3

/* ---- FP8 formats and scale granularities -------------------------------- */
#define B2Q_E4M3 0
#define B2Q_E5M2 1
#define B2Q_SCALE_CHANNEL  0   /* one scale per output row n:  [N]           */
#define B2Q_SCALE_TENSOR   1   /* one fp32 scalar, read on the device        */
#define B2Q_SCALE_BLOCK128 2   /* fp32 [ceil(N/128), ceil(K/128)]            */

/* ---- activation functions fused into grouped GEMM epilogues ------------- */
#define B2Q_ACT_NONE      0
#define B2Q_ACT_SILU_MUL  1    /* out[:, j] = silu(g[:, j]) * g[:, I + j]    */
#define B2Q_ACT_GELU_TANH_MUL 3 /* FP8 grouped GEMM only: out[:, j] = gelu_tanh(g[:, j]) * g[:, I + j]          */
#define B2Q_ACT_SILU_MUL_IN 2  /* INT4 grouped GEMM only: x has 2K columns (gate, then up; ldx >= 2K) and the
                                  GEMM's input row is silu(x[:, :K]) * x[:, K:], rounded to the activation type as
                                  B2Q_ACT_SILU_MUL would have stored it.  No output activation, no row_map.     */

B2Q_API const char* b2q_strerror(int code);
B2Q_API int b2q_version(void);
/* Compute capability check of the current device: 0 when it is sm_100. */
B2Q_API int b2q_device_ok(void);

/* ---- dequantisation (the bit-exactness gate) ----------------------------
 * out[N, K] (row-major, out_dtype) = round_to_out_dtype((q - 8) * scale).
 * Restates the unpack contract of tests/test_gemv_int4.py:172-210 and
 * tests/test_moe_int4_kernel.py:68-83.                                        */
B2Q_API int b2q_dequant_int4(const void* w, int w_layout, const void* scale, int scale_dtype,
                     void* out, int out_dtype, int64_t N, int64_t K, int group,
                     void* stream);
/* out[N, K] = decode(w[n,k]) * scale (fp32 math, one rounding to out_dtype).
 * tests/test_fp8_blockscale_gemm.py:31-36; patch test at
 * vllm/patches/vllm_for_multi_arc.patch:477-580.                              */
B2Q_API int b2q_dequant_fp8(const void* w, int fp8_format, const void* scale, int scale_dtype,
                    int scale_mode, void* out, int out_dtype, int64_t N, int64_t K,
                    void* stream);

/* Residual add + RMSNorm, the step the reference fuses in front of a decode GEMV
 * (esimd_resadd_norm_gemv_fp8_pert / _int4_pert / gemv2_fp8_pert, csrc/xpu/torch_extension.cc and
 * csrc/xpu/esimd_kernels/resadd_norm_gemv_int4.h, norm_gemv_fused.h):
 *   s = hidden + residual (fp32);  residual <- s;  normed_out <- s * rsqrt(mean(s^2) + eps) * norm_weight.
 * All tensors [M, K] contiguous in act_dtype (norm_weight [K]); K % 8 == 0.  The GEMV then runs on
 * normed_out through b2q_linear_fp8 / b2q_linear_int4; with kernel overlap on, its pre-pass and
 * weight stream start under this kernel.                                                       */
B2Q_API int b2q_resadd_rmsnorm(const void* hidden, void* residual, const void* norm_weight, void* normed_out,
                       int act_dtype, int64_t M, int64_t K, float eps, void* stream);

/* The general form behind b2q_resadd_rmsnorm, for the two further members of the family:
 *   v = hidden ? (hidden + residual) * scalar : residual        (fp32; with hidden, residual <- v)
 *   out1 = v * rsqrt(mean(v^2) + eps) * w1;   out2 = v * rsqrt(mean(v^2) + eps) * w2   (w2 / out2 both NULL or both set)
 * esimd_scaled_resadd_norm_gemv_fp8_pert (csrc/xpu/esimd_kernels/scaled_resadd_norm_gemv_fp8.h:70-95) is
 * hidden + scalar + one output followed by the FP8 GEMV; esimd_norm_gemv_norm_fp16
 * (csrc/xpu/esimd_kernels/norm_gemv_norm_fp16.h:56-98) is hidden = NULL with two weights, out1 feeding the
 * router GEMV and out2 being the MoE input.                                                              */
B2Q_API int b2q_rmsnorm_fused(const void* hidden, void* residual, float scalar, const void* w1, void* out1,
                      const void* w2, void* out2, int act_dtype, int64_t M, int64_t K, float eps, void* stream);

/* Gated RMSNorm, the step the reference fuses in front of the GDN out_proj GEMV
 * (esimd_norm_gemv_fp8_pert / _fp8_blockscale / _int4_pert, csrc/xpu/torch_extension.cc:117-121 and
 * csrc/xpu/esimd_kernels/norm_gemv_fused.h, norm_gemv_int4.h):  per row of x [rows, V]
 *   out = x * rsqrt(mean(x^2) + eps) * norm_weight * silu(z)   (fp32, one rounding to act_dtype).
 * x, z, out contiguous [rows, V], norm_weight [V].  The GEMV then runs on out viewed as [1, rows * V]. */
B2Q_API int b2q_gated_rmsnorm(const void* x, const void* z, const void* norm_weight, void* out, int act_dtype,
                      int64_t rows, int64_t V, float eps, void* stream);

/* GGML Q4_0 quantisation with group 128, the load-time step that produces b2q_linear_int4's inputs:
 * qweight int32 [M, K/8] (B2Q_W4_NMAJOR), scale fp16 [M, K/128] = signed group maximum / -8,
 * q = clamp(int(x / scale_fp32 + 8.5), 0, 15).  x is bf16 or fp16 [M, K] with row pitch ldx.
 * Replaces q4_0_quantize (csrc/xpu/torch_extension_q4_0.cc:29-84, csrc/xpu/q4_0_quant.sycl:29-125)
 * and follows that kernel's arithmetic step by step.  K % 128 == 0; rows 8-byte aligned.       */
B2Q_API int b2q_quantize_q4_0(const void* x, int act_dtype, int64_t ldx, void* qweight, void* scale_f16,
                      int64_t M, int64_t K, void* stream);

/* FP8 (e4m3) weight quantisation, the load-time step that produces b2q_linear_fp8's inputs:
 *   scale = max(amax, 1e-12) / 448 (fp32) per 128 x 128 block / per output row / per tensor (scale_mode, with the
 *   scale shapes of B2Q_SCALE_*), wq[n, k] = e4m3(w[n, k] / scale): fp32 division, one round-to-nearest-even.
 * w is bf16, fp16 or fp32 [N, K] with row pitch ldw (elements); wq is contiguous [N, K] bytes.  Ragged edge
 * blocks are allowed.  Follows the recipe of tests/test_fp8_blockscale_gemm.py:13-28 (block),
 * tests/test_fp8_blockscale_moe_prefill.py:18-51 and the per-channel / per-tensor scale rules of
 * vllm/patches/vllm_for_multi_arc.patch:477-580.                                                       */
B2Q_API int b2q_quantize_fp8(const void* w, int w_dtype, int64_t ldw, void* wq, float* scale, int scale_mode,
                     int64_t N, int64_t K, void* stream);

/* ---- dense weight-only linear: out[M, N] = x[M, K] * dequant(W)[N, K]^T --
 * fp32 accumulate, one rounding to act_dtype (x and out share act_dtype).
 * Replaces esimd_gemv_int4 / esimd_gemm_int4_pgrp
 * (csrc/xpu/torch_extension.cc:53-55, csrc/xpu/torch_extension_gemm.cc:20-22;
 *  kernels csrc/xpu/esimd_kernels/int4_GEMV.h:165-304, int4_GEMM.h:81-320).
 * Any M >= 1.  K % group == 0, group == 128, K % 8 == 0.
 * scale strides are in elements: scale(n, kg) = scale[n*s_stride_n + kg*s_stride_g].
 * ldx / ldo are row pitches of x / out in elements.
 * workspace is optional (NULL / 0 allowed).  With at least b2q_linear_workspace_bytes() of
 * scratch the tensor-core kernel first rewrites the activations as fp16 times a per-token power
 * of two in the element order its nibble decode produces; the dequantised weight is then
 * (q - 8) * scale rounded once to fp16 (11 significant bits) instead of to the activation type.
 * Scales of any magnitude are safe on that route: bf16 / fp32 scales are brought into fp16's normal
 * range by a power of two per output row, chosen from the row's first group of the K range a CTA
 * works on and taken out of the fp32 accumulator again.  Groups within 2^13 of that first one, either
 * way, are exact; a group further below loses bits, one further above is saturated and reported
 * through b2q_device_status (code 109).
 * Without scratch the weight is rounded exactly as the torch reference rounds it.  For M <= 64
 * the scratch also holds partial sums: layers with few output rows are cut along K over several CTAs
 * per strip of rows so that they still occupy every SM; the partial sums are added in a fixed order,
 * so results are bit-reproducible from run to run.                                              */
B2Q_API size_t b2q_linear_workspace_bytes(int64_t M, int64_t N, int64_t K);
B2Q_API int b2q_linear_int4(const void* x, int act_dtype, int64_t ldx,
                    const void* w, int w_layout,
                    const void* scale, int scale_dtype, int64_t s_stride_n, int64_t s_stride_g,
                    void* out, int64_t ldo,
                    int64_t M, int64_t N, int64_t K, int group,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Replaces esimd_gemv_fp8_pern / esimd_gemv_fp8_pert / esimd_gemm_fp8_pert /
 * esimd_gemm_fp8_blockscale (csrc/xpu/torch_extension.cc:9-37,
 * csrc/xpu/torch_extension_gemm.cc:14-28; kernels fp8_GEMV_v2.h:46-403,
 * fp8_GEMM_pert.h:4030-4075, fp8_GEMM_blockscale.h:64-223).
 * w is [N, K] one byte per element, row-major.  Activation stays 16-bit
 * (w8a16); e4m3 decode is exact including subnormals.  K % 16 == 0.
 * workspace is optional (NULL / 0 allowed).  With at least
 * b2q_linear_fp8_workspace_bytes() of scratch:
 *  - M <= 64 with per-channel or per-tensor scales runs on the 8-bit tensor-core path: the weights are
 *    used as stored and every activation row is rewritten as 2^e times a sum of two (bf16) or three
 *    (fp16) e4m3 terms, which reproduces it exactly (elements more than 2^14 below their row maximum
 *    lose low bits);
 *  - otherwise bf16 activations are rewritten as fp16 times a per-token power of two (exact for every
 *    element within 2^-31 of its row maximum), which makes the in-kernel fp8 decode four times cheaper. */
B2Q_API size_t b2q_linear_fp8_workspace_bytes(int64_t M, int64_t N, int64_t K);
B2Q_API int b2q_linear_fp8(const void* x, int act_dtype, int64_t ldx,
                   const void* w, int fp8_format,
                   const void* scale, int scale_dtype, int scale_mode,
                   void* out, int64_t ldo,
                   int64_t M, int64_t N, int64_t K,
                   void* workspace, size_t workspace_bytes, void* stream);

/* Residual add + RMSNorm + FP8 weight-only linear as one call (esimd_resadd_norm_gemv_fp8_pert,
 * esimd_scaled_resadd_norm_gemv_fp8_pert: csrc/xpu/esimd_kernels/norm_gemv_fused.h,
 * scaled_resadd_norm_gemv_fp8.h:70-95):
 *   v = (hidden + residual) * scalar;  residual <- v;  normed_out <- v * rsqrt(mean(v^2) + eps) * norm_weight;
 *   out = normed_out * dequant(W)^T            (normed_out as stored, i.e. rounded to act_dtype).
 * hidden, residual, normed_out are contiguous [M, K], norm_weight [K]; the rest as b2q_linear_fp8.  On the decode
 * path (M <= 64, per-channel or per-tensor scale, scratch given) the norm runs inside the GEMV's own activation
 * pre-pass: two launches in all (pre-pass, GEMV) instead of three; elsewhere the norm is its own launch.          */
B2Q_API int b2q_resadd_norm_linear_fp8(const void* hidden, void* residual, const void* norm_weight, void* normed_out,
                               float eps, float scalar, int act_dtype, const void* w, int fp8_format,
                               const void* scale, int scale_dtype, int scale_mode, void* out, int64_t ldo,
                               int64_t M, int64_t N, int64_t K, void* workspace, size_t workspace_bytes, void* stream);

/* Per-token, per-128-column dynamic e4m3 quantisation of activations:
 * xs[m, kb] = max(amax(x[m, 128kb:128kb+128]), 1e-12) / 448 ; xq = e4m3(x / xs).
 * (the (1,128) dynamic activation key of
 *  vllm/patches/vllm_for_multi_arc.patch:2628-2634)                           */
B2Q_API int b2q_act_quant_fp8_1x128(const void* x, int act_dtype, int64_t ldx,
                            void* xq, float* xs, int64_t M, int64_t K, void* stream);

/* W8A8 block-scaled GEMM: out = dq(xq, xs) * dq(w, ws)^T, e4m3 x e4m3 tensor
 * cores, fp32 promotion per 128-deep K block.  Same weight contract as
 * esimd_gemm_fp8_blockscale.  M, N arbitrary; K % 128 == 0.                   */
B2Q_API int b2q_gemm_fp8_block_w8a8(const void* xq, const float* xs,
                            const void* w, const float* ws,
                            void* out, int out_dtype, int64_t ldo,
                            int64_t M, int64_t N, int64_t K, void* stream);

/* ---- MoE routing ---------------------------------------------------------
 * softmax over E in fp32 -> top_k rounds of (max, lowest index among equal)
 * -> optional renormalisation.  weights[T, k] in w_dtype, ids[T, k] int32.
 * Replaces esimd_moe_topk / topk_v2 / moe_topk_int4 / moe_topk_softmax
 * (csrc/xpu/esimd_kernels/moe_ops.h:106-231).  E <= 1024, top_k <= 32.         */
B2Q_API int b2q_moe_topk(const void* logits, int logits_dtype, int64_t T, int E, int top_k,
                 int renorm, void* weights, int w_dtype, int32_t* ids, void* stream);

/* Counting sort of the T*k (token, slot) pairs by expert id; stable in pair
 * index.  expert_offsets has E+1 entries (exclusive prefix, last = T*k);
 * expert_tokens[pos] = pair index; pair_to_perm[pair] = pos (may be NULL);
 * rows_per_expert[E] (may be NULL).  Replaces moe_prefill_gather_forward_v2
 * (csrc/moe_prefill/moe_prefill_int4.sycl:40-106, 458-488) and the atomic
 * scatter of moe_ops.h:437-569.  workspace: b2q_moe_route_workspace_bytes().   */
B2Q_API size_t b2q_moe_route_workspace_bytes(int64_t n_pairs, int E);
B2Q_API int b2q_moe_route(const int32_t* ids, int64_t n_pairs, int E,
                  int32_t* expert_offsets, int32_t* expert_tokens,
                  int32_t* pair_to_perm, int32_t* rows_per_expert,
                  void* workspace, size_t workspace_bytes, void* stream);

/* Same sort, same outputs, no workspace argument.  This entry point has no counterpart in
 * the reference.  It is for callers that must not allocate device memory around the call:
 * code running inside a stream capture (where cudaMalloc is not allowed), runtimes that plan
 * all device memory in advance, hosts without a pooled allocator.  The scratch table lives in
 * a fixed array inside the library (256 KB per GPU that loads it, held until exit), so
 *   - n_pairs <= 65536 and E <= 256, otherwise B2Q_ERR_LIMIT;
 *   - the first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture;
 *   - every call on a device uses the same array: calls whose kernels may overlap on the GPU
 *     (different streams) race on it.  Nothing needs clearing between calls.
 * It calls no allocation routine of any kind.                                               */
B2Q_API int b2q_moe_route_static(const int32_t* ids, int64_t n_pairs, int E,
                  int32_t* expert_offsets, int32_t* expert_tokens,
                  int32_t* pair_to_perm, int32_t* rows_per_expert, void* stream);

/* dst[r, :] = src[idx[r] / div, :] for r < rows (row gather; div = top_k maps
 * pair index -> token).  Replaces moe_prefill_scatter_x_forward (:818-859).   */
B2Q_API int b2q_gather_rows(const void* src, const int32_t* idx, int div, void* dst,
                    int64_t rows, int64_t cols, int elem_bytes, void* stream);

/* out[r, j] = silu(in[r, j]) * in[r, I + j], fp32 math.
 * Replaces esimd_moe_silu_mul (moe_ops.h:576-621).                            */
B2Q_API int b2q_silu_mul(const void* in, void* out, int dtype, int64_t rows, int64_t I, void* stream);

/* out[r, j] = gelu_tanh(in[r, j]) * in[r, I + j] with gelu_tanh(g) = 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))),
 * fp32 math, one rounding.  Replaces esimd_moe_gelu_tanh_mul (csrc/xpu/torch_extension_moe.cc:30-34,
 * csrc/xpu/esimd_kernels/moe_ops.h:678-740).                                  */
B2Q_API int b2q_gelu_tanh_mul(const void* in, void* out, int dtype, int64_t rows, int64_t I, void* stream);

/* out[t, :] = sum_s w[t, s] * y[perm ? perm[t*k+s] : t*k+s, :], fp32 sum.
 * w == NULL adds the rows unweighted (moe_ops.moe_accumulate, csrc/moe_batch/moe.sycl:1177-1230);
 * with top_k == 1, perm == NULL and out == y it scales row t by w[t] in place (the routing-weight
 * multiply of moe_down_fp8_grouped, csrc/moe_batch/moe_fp8_grouped.h:293-335).
 * w_by_row != 0 reads the weight at the row position instead of at (t, s).
 * Replaces moe_prefill_accumulate{,_permuted}_forward_v2 (:398-454) and
 * esimd_moe_gather (moe_ops.h:627-676).                                       */
B2Q_API int b2q_moe_combine(const void* y, const void* w, int w_dtype, const int32_t* perm,
                    void* out, int dtype, int64_t T, int top_k, int64_t H, int w_by_row, void* stream);

/* Tail of the decode pipeline with a shared expert (moe_forward_full_int4,
 * csrc/moe_batch/moe_int4.sycl:3086-3166: gate precompute, shared down scaled by the gate, accumulate):
 *   out[t, :] = routed[t, :] + sigmoid(x[t, :] . gate_w[:]) * shared[t, :]   (fp32, one rounding).
 * x, shared, routed, out contiguous [T, H] in dtype, gate_w [H]; H % 8 == 0; out may alias routed.   */
B2Q_API int b2q_moe_shared_gate_add(const void* x, const void* gate_w, const void* shared, const void* routed,
                            void* out, int dtype, int64_t T, int64_t H, void* stream);

/* ---- MoE grouped GEMMs ----------------------------------------------------
 * Rows [expert_offsets[e], expert_offsets[e+1]) of the (virtual) expert-sorted
 * input use expert e's weight.  If row_map != NULL the input row of sorted row
 * r is x[row_map[r] / row_div]; otherwise it is x[r].  Output row r is written
 * at out[out_map ? out_map[r] : r].  act = B2Q_ACT_SILU_MUL treats the weight
 * as [gate rows ; up rows] (N = 2*I) and writes I columns.
 * INT4: w is E stacked matrices in w_layout, scales E stacked.
 * Replaces moe_prefill_up/down_forward_v2 (:493-621), moe_gemm_int4_nmajor
 * (csrc/moe_batch/moe_int4.sycl:3373-3552).                                    */
/* gather is ignored (kept for call compatibility): the pre-passed activations are always staged. */
B2Q_API size_t b2q_moe_gemm_workspace_bytes(int64_t rows, int E, int64_t N, int64_t K, int act, int gather);
B2Q_API int b2q_moe_gemm_int4(const void* x, int act_dtype, int64_t ldx,
                      const int32_t* row_map, int row_div,
                      const void* w, int w_layout, const void* scale, int scale_dtype,
                      const int32_t* expert_offsets, int E,
                      void* out, int64_t ldo, const int32_t* out_map,
                      int64_t rows, int64_t N, int64_t K, int group, int act,
                      void* workspace, size_t workspace_bytes, void* stream);
/* FP8 e4m3 [E, N, K] with scale_mode CHANNEL ([E,N] fp32), TENSOR ([E] fp32)
 * or BLOCK128 ([E, ceil(N/128), ceil(K/128)] fp32).  Replaces
 * esimd_moe_gemm_fp8{,_pert,_blockscale} (csrc/xpu/torch_extension_moe.cc:41-56).*/
B2Q_API int b2q_moe_gemm_fp8(const void* x, int act_dtype, int64_t ldx,
                     const int32_t* row_map, int row_div,
                     const void* w, int fp8_format, const float* scale, int scale_mode,
                     const int32_t* expert_offsets, int E,
                     void* out, int64_t ldo, const int32_t* out_map,
                     int64_t rows, int64_t N, int64_t K, int act,
                     void* workspace, size_t workspace_bytes, void* stream);

/* ---- sum of row-parallel partial results over the GPUs of one box ----------------------------
 * The exchange step behind a row-parallel linear (o_proj, down) of a tensor-parallel decoder layer; the
 * reference calls the serving framework's all-reduce there (vllm/patches/vllm_for_multi_arc.patch:10185,
 * :10199, :8006-8010).  One communicator per rank and per tile shape bound (max_rows x max_cols 16-bit
 * values).  b2q_comm_create allocates the rank's buffer (cudaMalloc: set-up time only, the one place this
 * library allocates) and returns its 64-byte CUDA IPC handle; the caller gathers the handles of all ranks
 * (rank order) and passes them to b2q_comm_connect.  b2q_allreduce_sum then launches ONE kernel on the
 * caller's stream: partial columns go to their owner rank by plain peer stores, the owner adds the `world`
 * partial tiles in rank order in fp32 (all ranks get bit-identical results), rounds once and stores the
 * sum into every rank's buffer; flags with a call epoch order the steps, every wait on a flag is bounded
 * by wait_limit_ms (<= 0: two seconds) and an expired wait is reported by b2q_comm_status (the
 * communicator must then be re-created on all ranks).  *out receives the DEVICE address of the [M, N]
 * result inside this rank's buffer (row pitch N); it stays valid until the next call but one.
 * All ranks must call with the same M, N, dtype, in the same order.  N % (8 * world) == 0, N / world <=
 * 65536, M <= max_rows <= 4096.  No multicast, no library collective, no allocation per call.
 * Two forms of the same sum, chosen when the communicator is made (the same on all ranks):
 *   B2Q_COMM_TWO_STEPS  the form described above: bytes per rank independent of world
 *   B2Q_COMM_ONE_STEP   every rank stores its whole tile into every rank's buffer and every rank adds the world
 *                       tiles itself (rank order, fp32): one trip over the links instead of two, world - 1 times
 *                       the bytes; needs N <= 65536
 *   B2Q_COMM_AUTO       one step while (world - 1) * max_rows * max_cols * 2 bytes <= 8 MiB (decode tiles on
 *                       any number of ranks), two steps otherwise; b2q_comm_create uses this             */
#define B2Q_COMM_AUTO 0
#define B2Q_COMM_ONE_STEP 1
#define B2Q_COMM_TWO_STEPS 2
B2Q_API int b2q_comm_create(int rank, int world, int64_t max_rows, int64_t max_cols, void** comm, void* ipc_handle_out);
B2Q_API int b2q_comm_create_mode(int rank, int world, int64_t max_rows, int64_t max_cols, int mode, void** comm, void* ipc_handle_out);
B2Q_API int b2q_comm_connect(void* comm, const void* all_ipc_handles /* world x 64 bytes */);
B2Q_API int b2q_comm_destroy(void* comm);
B2Q_API int b2q_comm_status(void* comm, int* out);
/* Device address of result area `which` (0 or 1; calls alternate between the two, starting with 0).  */
B2Q_API int b2q_comm_result_ptr(void* comm, int which, void** out);
B2Q_API int b2q_allreduce_sum(void* comm, const void* in, int dtype, int64_t ldi, int64_t M, int64_t N,
                      double wait_limit_ms, void** out, void* stream);
/* Row-parallel INT4 linear and the sum of its partial results as one call: out = sum over ranks of
 * x_r[M, K_r] * dequant(W_r)[N, K_r]^T.  Same arguments as b2q_linear_int4; `partial` is [M, N] scratch in
 * act_dtype (row pitch ldp).  For decode tiles (8 < M <= 64, N % (128 * world) == 0) the GEMM's epilogue
 * itself stores each 128-column strip of its result into the owner rank's reduction slot over NVLink and
 * raises that strip's flag, so the exchange starts while other strips are still being computed and the
 * partial tile never goes through local memory; the reduction kernel that follows only adds and
 * publishes.  Other shapes run the plain GEMM into `partial` followed by b2q_allreduce_sum.  *out as in
 * b2q_allreduce_sum.  Replaces the row-parallel linear + all-reduce pairs of
 * vllm/patches/vllm_for_multi_arc.patch:10185, :10199.                                                   */
B2Q_API int b2q_linear_int4_allreduce(const void* x, int act_dtype, int64_t ldx, const void* w, int w_layout,
                              const void* scale, int scale_dtype, int64_t s_stride_n, int64_t s_stride_g,
                              void* partial, int64_t ldp, int64_t M, int64_t N, int64_t K, int group,
                              void* workspace, size_t workspace_bytes, void* comm, double wait_limit_ms,
                              void** out, void* stream);
/* The same protocol with all `world` ranks living in ONE process on ONE device, for tests on a single GPU:
 * b2q_comm_connect_local wires communicators created with ipc_handle_out == NULL to one another, and
 * b2q_allreduce_sum_emulated runs the first n_present ranks as one cooperative launch (ranks wait for one
 * another, so they may not be separate launches on one GPU).  n_present < world makes the present ranks'
 * waits run out after wait_limit_ms: the give-up path, exercised without a hang.                      */
B2Q_API int b2q_comm_connect_local(void** comms, int world);
B2Q_API int b2q_allreduce_sum_emulated(void** comms, int world, int n_present, const void* const* ins, int dtype,
                               int64_t ldi, int64_t M, int64_t N, double wait_limit_ms, void** outs, void* stream);

/* ---- token exchange of an expert-parallel MoE layer over the GPUs of one box ---------------------------
 * The reference splits the experts contiguously over the ranks (vllm/patches/vllm_for_multi_arc.patch:3356-3365)
 * and emulates the all-to-all with an all-gather and a reduce-scatter of the whole batch (:1559-1563).  Here the
 * rows travel by plain peer stores and every count stays on the device (a library all-to-all wants the counts on
 * the host first).  One communicator per rank; cap_rows = the most (token, slot) pairs one rank sends in a pass
 * (its tokens x top_k), H = row width in 16-bit values (H % 8 == 0).  Set-up as for b2q_comm_create: the
 * communicator allocates its buffer (the receive area [world x cap_rows x H], the expert indices of those rows
 * [world x cap_rows] int32, the return area [cap_rows x H]) and hands out a 64-byte CUDA IPC handle; gather the
 * handles in rank order and pass them to b2q_ep_connect.  One pass, all calls on one stream:
 *   b2q_ep_dispatch  x [T, ldx]; order[n_pairs] = pair indices (token * top_k + slot) sorted by destination rank,
 *                    dest_offsets[world + 1] = where each rank's segment starts (both from b2q_moe_route over
 *                    expert / experts_per_rank with `world` buckets), local_ids[n_pairs] = expert index on the
 *                    owner, in the same order.  Copies the rows into slot `rank` of every owner's receive area;
 *                    unused positions of the slot get the index -1 (b2q_moe_route drops those).
 *   b2q_ep_wait(0)   returns on the stream once the slots of all ranks have landed here.  The caller then routes
 *                    the world * cap_rows indices and runs the grouped GEMMs over the receive area with
 *                    rows = world * cap_rows as an upper bound; results go back to the rows' positions.
 *   b2q_ep_return    y [world * cap_rows, ldy] in receive-area order: every filled row goes to its source rank's
 *                    return area at the position it had in that rank's `order`.
 *   b2q_ep_wait(1)   returns once all owners' results have landed; the return area then holds [n_pairs, H] in
 *                    `order` order, ready for b2q_moe_combine.
 * Waits are bounded by wait_limit_ms (<= 0: two seconds); an expired wait is reported by b2q_ep_status (301: rows
 * missing, 302: results missing) and the communicators must then be re-created on all ranks.  All ranks make the
 * same calls in the same order.  No multicast, no library collective, no allocation and no host read per pass.
 * b2q_ep_connect_local wires communicators of ONE process on ONE device (tests): run each step for all ranks
 * before the next step, so that no kernel waits for a later launch.                                      */
B2Q_API int b2q_ep_create(int rank, int world, int64_t cap_rows, int64_t H, void** comm, void* ipc_handle_out);
B2Q_API int b2q_ep_connect(void* comm, const void* all_ipc_handles /* world x 64 bytes */);
B2Q_API int b2q_ep_connect_local(void** comms, int world);
B2Q_API int b2q_ep_destroy(void* comm);
B2Q_API int b2q_ep_status(void* comm, int* out);
B2Q_API int b2q_ep_buffers(void* comm, void** recv_rows, void** recv_ids, void** ret_rows);
B2Q_API int b2q_ep_dispatch(void* comm, const void* x, int dtype, int64_t ldx, const int32_t* order, int top_k,
                    const int32_t* dest_offsets, const int32_t* local_ids, int64_t n_pairs, void* stream);
B2Q_API int b2q_ep_return(void* comm, const void* y, int dtype, int64_t ldy, void* stream);
B2Q_API int b2q_ep_wait(void* comm, int phase, double wait_limit_ms, void* stream);

/* Code of the first bounded device-side wait that expired since the library was loaded
 * (0 = none).  Synchronises the device; meant for tests and post-mortems.       */
B2Q_API int b2q_device_status(int* out);
/* Clears that code on the current device: the status words of every kernel family, and the arrival
 * counters of strips cut between CTAs (a CTA that gave up never delivered its arrival, so a stale
 * counter would make a later launch finish that strip early).  Synchronises the device first; call
 * it with no launch of this library in flight, once per device that reported a code.           */
B2Q_API int b2q_device_status_reset(void);
/* Self-test of the bounded waits: launches one CTA that waits, with a limit of about a millisecond,
 * on a barrier nobody arrives on.  The wait gives up, records `code` (> 0) as the device status and
 * writes 1 to *gave_up (a DEVICE int); the context stays usable.  Nothing faults or hangs.       */
B2Q_API int b2q_selftest_bounded_wait(int code, int* gave_up, void* stream);

/* Kernel selection override for benchmarking: 0 = automatic, 1 = the mma.sync streaming kernel,
 * 2 = the tcgen05 kernel with 16-bit operands, 3 = the same without activation pre-pass,
 * 4 = the same with one CTA per strip (no strip cutting), 5 = INT4 decode on the int8 MMA,
 * 6 = the CTA-pair (cta_group::2) variant of the W8A8 GEMM.                                  */
B2Q_API void b2q_set_force_kernel(int which);
/* Overlap of consecutive kernels on a stream (programmatic dependent launch), per calling thread:
 *   0  off: every kernel starts after the one before it has completed.
 *   1  (default) the activation pre-pass and the GEMM of one call overlap: the GEMM streams and
 *      converts weights while the pre-pass runs, and waits for it before it reads activations.
 *   2  additionally declares the weight and scale tensors static: no kernel that precedes a b2q
 *      call on its stream writes them.  A GEMM may then start streaming weights while the kernels
 *      before it (the previous layer) are still draining.  Activations, outputs and scratch stay
 *      fully ordered in every mode.                                             */
B2Q_API void b2q_set_overlap_mode(int mode);
/* Name of the kernel family the last b2q_linear_* / b2q_moe_gemm_* call on this
 * thread launched ("smallm", "umma", ...).                                    */
B2Q_API const char* b2q_last_kernel(void);
/* Number of kernel launches issued by this library on this thread so far.     */
B2Q_API uint64_t b2q_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B2Q_H_ */
