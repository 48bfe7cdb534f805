// torch custom-op registration of the dense decode / prefill linears in C++, for the CUDA dispatch key, straight over the
// C ABI of include/b2q.h.  The reference registers the same names for the XPU key in its C++ registration units
// (csrc/xpu/torch_extension.cc:9-61, csrc/xpu/torch_extension_gemm.cc:14-37); its Python package only forwards to
// torch.ops.  An eager call of these ops therefore costs one dispatcher hop and the launches, not a Python function,
// a ctypes marshalling and a second Python frame (measured on the [16 x 4096 x 4096] INT4 linear: 24 us per eager call
// through the Python registration, of which the kernel is 10).
//
// Built by build.py into custom_esimd_kernels_vllm/libb2q_torch.so, which links libb2q.so and libtorch.  Only
// TORCH_LIBRARY_IMPL blocks live here: the schemas are defined once, by the Python registration module, which skips
// its own implementation for the names this library reports through b2q_torch_ops().  The checks and their messages
// are those of the Python implementation (custom_esimd_kernels_vllm/_impl.py: linear_int4, linear_fp8).
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include "b2q.h"

namespace {

constexpr int64_t GROUP = 128;

int act_dtype(const at::Tensor& t) {
  if (t.scalar_type() == at::kBFloat16) return B2Q_BF16;
  if (t.scalar_type() == at::kHalf) return B2Q_F16;
  if (t.scalar_type() == at::kFloat) return B2Q_F32;
  TORCH_CHECK(false, "b2q: unsupported dtype ", t.scalar_type());
}

void require_cuda(std::initializer_list<const at::Tensor*> ts) {
  for (const at::Tensor* t : ts) TORCH_CHECK(t->is_cuda(), "b2q: tensor must live on a CUDA device (no CPU path exists)");
}

void check(int rc) { TORCH_CHECK(rc == 0, b2q_strerror(rc)); }

at::Tensor scratch(size_t bytes, const at::Tensor& like) {
  return at::empty({(int64_t)bytes}, like.options().dtype(at::kByte));      // caching allocator: no cudaMalloc in steady state
}

// The INT4 presentations of custom_esimd_kernels_vllm/_impl.py::_int4_view: uint8 [N, K/2] or int32 [N, K/8] contiguous
// (N-major), the .t() view of the latter, or int32 [K/8, N] contiguous with scales [K/128, N] (K-major).
struct Int4View { const void* w; int layout; int64_t N, K, sn, sg; };

Int4View int4_view(const at::Tensor& weight, const at::Tensor& scale) {
  TORCH_CHECK(weight.dim() == 2 && scale.dim() == 2, "int4 weight and scale must be 2-D");
  Int4View v{};
  v.w = weight.data_ptr();
  if (weight.scalar_type() == at::kByte) {
    TORCH_CHECK(weight.is_contiguous(), "uint8 int4 weight must be contiguous [N, K/2]");
    v.N = weight.size(0); v.K = weight.size(1) * 2; v.layout = B2Q_W4_NMAJOR;
  } else if (weight.scalar_type() == at::kInt) {
    const int64_t a = weight.size(0), b = weight.size(1);
    if (!weight.is_contiguous() && weight.stride(0) == 1 && weight.stride(1) == a) {
      v.N = b; v.K = a * 8; v.layout = B2Q_W4_NMAJOR;
    } else {
      TORCH_CHECK(weight.is_contiguous(), "int4 weight must be contiguous or a transposed view of a contiguous tensor");
      const bool nmaj = scale.size(0) == a && scale.size(1) * GROUP == b * 8;
      const bool kmaj = scale.size(1) == b && scale.size(0) * GROUP == a * 8;
      if (nmaj || !kmaj) { v.N = a; v.K = b * 8; v.layout = B2Q_W4_NMAJOR; }
      else { v.N = b; v.K = a * 8; v.layout = B2Q_W4_KMAJOR; }
    }
  } else {
    TORCH_CHECK(false, "int4 weight must be uint8 or int32, got ", weight.scalar_type());
  }
  TORCH_CHECK(v.K % GROUP == 0, "K must be a multiple of the group size 128");
  const int64_t G = v.K / GROUP;
  if (scale.size(0) == v.N && scale.size(1) == G) { v.sn = scale.stride(0); v.sg = scale.stride(1); }
  else if (scale.size(0) == G && scale.size(1) == v.N) { v.sn = scale.stride(1); v.sg = scale.stride(0); }
  else TORCH_CHECK(false, "int4 scale shape [", scale.size(0), ", ", scale.size(1), "] does not match N=", v.N, ", K/128=", G);
  return v;
}

at::Tensor linear_int4(const at::Tensor& input, const at::Tensor& weight, const at::Tensor& weight_scale, at::Tensor output) {
  require_cuda({&input, &weight, &weight_scale, &output});
  TORCH_CHECK(input.dim() == 2 && output.dim() == 2, "input/output must be 2-D");
  TORCH_CHECK(input.scalar_type() == at::kBFloat16 || input.scalar_type() == at::kHalf, "activation must be bf16 or fp16");
  TORCH_CHECK(output.scalar_type() == input.scalar_type(), "output dtype must equal input dtype");
  const Int4View v = int4_view(weight, weight_scale);
  const int64_t M = input.size(0);
  TORCH_CHECK(input.size(1) == v.K, "input K does not match weight");
  TORCH_CHECK(output.size(0) == M && output.size(1) == v.N, "output must be [M, N]");
  TORCH_CHECK(input.stride(1) == 1 && output.stride(1) == 1, "input/output rows must be contiguous");
  const c10::cuda::CUDAGuard guard(input.device());
  const size_t wsb = b2q_linear_workspace_bytes(M, v.N, v.K);
  const at::Tensor ws = scratch(wsb, input);
  check(b2q_linear_int4(input.data_ptr(), act_dtype(input), M > 1 ? input.stride(0) : v.K, v.w, v.layout,
                        weight_scale.data_ptr(), act_dtype(weight_scale), v.sn, v.sg, output.data_ptr(),
                        M > 1 ? output.stride(0) : v.N, M, v.N, v.K, (int)GROUP, wsb ? ws.data_ptr() : nullptr, wsb,
                        c10::cuda::getCurrentCUDAStream(input.device().index()).stream()));
  return output;
}

int fp8_format(const at::Tensor& w) {
  if (w.scalar_type() == at::kFloat8_e5m2) return B2Q_E5M2;
  if (w.scalar_type() == at::kFloat8_e4m3fn || w.scalar_type() == at::kByte || w.scalar_type() == at::kChar) return B2Q_E4M3;
  TORCH_CHECK(false, "b2q: fp8 weight must be float8_e4m3fn / float8_e5m2 / uint8, got ", w.scalar_type());
}

at::Tensor linear_fp8(const at::Tensor& input, const at::Tensor& weight, const at::Tensor& weight_scale, at::Tensor output,
                      int scale_mode, int64_t N, int64_t K) {
  require_cuda({&input, &weight, &weight_scale, &output});
  TORCH_CHECK(input.dim() == 2 && output.dim() == 2 && weight.dim() == 2, "input/weight/output must be 2-D");
  TORCH_CHECK(input.scalar_type() == at::kBFloat16 || input.scalar_type() == at::kHalf, "activation must be bf16 or fp16");
  TORCH_CHECK(output.scalar_type() == input.scalar_type(), "output dtype must equal input dtype");
  TORCH_CHECK(weight.is_contiguous(), "fp8 weight must be a contiguous [N, K] tensor (a transposed view is read wrongly)");
  const int64_t wn = weight.size(0), wk = weight.size(1), M = input.size(0);
  TORCH_CHECK((N < 0 || N == wn) && (K < 0 || K == wk), "N/K do not match the weight shape");
  TORCH_CHECK(input.size(1) == wk && output.size(0) == M && output.size(1) == wn, "shape mismatch");
  TORCH_CHECK(input.stride(1) == 1 && output.stride(1) == 1, "input/output rows must be contiguous");
  if (scale_mode == B2Q_SCALE_CHANNEL) {
    TORCH_CHECK(weight_scale.numel() == wn && weight_scale.is_contiguous(), "per-channel scale must have N elements");
  } else if (scale_mode == B2Q_SCALE_TENSOR) {
    TORCH_CHECK(weight_scale.numel() == 1 && weight_scale.scalar_type() == at::kFloat, "per-tensor scale must be one fp32");
  } else {
    TORCH_CHECK(weight_scale.scalar_type() == at::kFloat && weight_scale.is_contiguous(), "block scale must be fp32");
    TORCH_CHECK(weight_scale.dim() == 2 && weight_scale.size(0) == (wn + 127) / 128 && weight_scale.size(1) == (wk + 127) / 128,
                "block scale shape mismatch");
  }
  const c10::cuda::CUDAGuard guard(input.device());
  size_t wsb = 0;
  at::Tensor ws;
  if (input.scalar_type() == at::kBFloat16 || M <= 64) {
    wsb = b2q_linear_fp8_workspace_bytes(M, wn, wk);
    ws = scratch(wsb, input);
  }
  check(b2q_linear_fp8(input.data_ptr(), act_dtype(input), M > 1 ? input.stride(0) : wk, weight.data_ptr(), fp8_format(weight),
                       weight_scale.data_ptr(), act_dtype(weight_scale), scale_mode, output.data_ptr(),
                       M > 1 ? output.stride(0) : wn, M, wn, wk, wsb ? ws.data_ptr() : nullptr, wsb,
                       c10::cuda::getCurrentCUDAStream(input.device().index()).stream()));
  return output;
}

at::Tensor gemv_int4(const at::Tensor& input, const at::Tensor& weight, const at::Tensor& weight_scale, at::Tensor output) {
  return linear_int4(input, weight, weight_scale, output);
}
at::Tensor gemv_fp8_pern(const at::Tensor& input, const at::Tensor& weight, const at::Tensor& weight_scale, at::Tensor output,
                         int64_t N, int64_t K) {
  return linear_fp8(input, weight, weight_scale, output, B2Q_SCALE_CHANNEL, N, K);
}
at::Tensor fp8_pert(const at::Tensor& input, const at::Tensor& weight, const at::Tensor& weight_scale, at::Tensor output) {
  return linear_fp8(input, weight, weight_scale, output, B2Q_SCALE_TENSOR, -1, -1);
}
at::Tensor fp8_blockscale(const at::Tensor& input, const at::Tensor& weight, const at::Tensor& weight_scale, at::Tensor output,
                          int64_t block_n, int64_t block_k) {
  TORCH_CHECK(block_n == 128 && block_k == 128, "only block_n == block_k == 128 is supported");
  return linear_fp8(input, weight, weight_scale, output, B2Q_SCALE_BLOCK128, -1, -1);
}

const char* const kOps =
    "esimd_gemv_int4,esimd_gemm_int4_pgrp,esimd_gemv_fp8_pern,esimd_gemv_fp8_pert,esimd_gemv_fp8_pert_bmg,"
    "esimd_gemm_fp8_pert,esimd_gemm_fp8_blockscale";

}  // namespace

// Names (comma separated, namespace custom_esimd_kernels_vllm) this library implements for the CUDA key.
extern "C" __attribute__((visibility("default"))) const char* b2q_torch_ops() { return kOps; }

TORCH_LIBRARY_IMPL(custom_esimd_kernels_vllm, CUDA, m) {
  m.impl("esimd_gemv_int4", &gemv_int4);
  m.impl("esimd_gemm_int4_pgrp", &gemv_int4);
  m.impl("esimd_gemv_fp8_pern", &gemv_fp8_pern);
  m.impl("esimd_gemv_fp8_pert", &fp8_pert);
  m.impl("esimd_gemv_fp8_pert_bmg", &fp8_pert);
  m.impl("esimd_gemm_fp8_pert", &fp8_pert);
  m.impl("esimd_gemm_fp8_blockscale", &fp8_blockscale);
}
