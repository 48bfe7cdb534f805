"""CPU oracle (test infrastructure only) of the residual-add + RMSNorm front end of the reference's fused decode
GEMVs, restating the step-by-step check of tests/test_resadd_norm_gemv_int4.py:41-59:
    s = hidden + residual (fp32);  residual' = s -> 16 bit;  normed = s * rsqrt(mean(s^2) + eps) * weight -> 16 bit.
The GEMV that follows consumes `normed` as stored (16 bit), through oracle.int4.linear / oracle.fp8.linear_tensor.
"""
import torch


def resadd_rmsnorm(hidden: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float):
    dt = hidden.dtype
    s = hidden.float() + residual.float()
    inv = torch.rsqrt(s.pow(2).mean(dim=-1, keepdim=True) + eps)
    normed = s * inv * norm_weight.float()
    return s.to(dt), normed.to(dt)


def gated_rmsnorm(x: torch.Tensor, z: torch.Tensor, norm_weight: torch.Tensor, eps: float):
    """rmsnorm(x) * norm_weight * silu(z) per row in fp32, one rounding; returns [1, rows * V]
    (tests/test_fp8_blockscale_fusions.py:91-96)."""
    xf = x.float()
    n = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    n = n * norm_weight.float() * torch.nn.functional.silu(z.float())
    return n.to(x.dtype).flatten().unsqueeze(0)


def scaled_resadd_rmsnorm(hidden, residual, norm_weight, eps, scalar):
    """v = (hidden + residual) * scalar in fp32; residual' = v -> 16 bit; normed = v * rsqrt(mean(v^2) + eps) * weight
    (csrc/xpu/esimd_kernels/scaled_resadd_norm_gemv_fp8.h:70-95)."""
    dt = hidden.dtype
    v = (hidden.float() + residual.float()) * scalar
    inv = torch.rsqrt(v.pow(2).mean(dim=-1, keepdim=True) + eps)
    return v.to(dt), (v * inv * norm_weight.float()).to(dt)


def norm_two_scales(residual, w1, w2, eps):
    """One 1/rms of the row, two post-norm scales (csrc/xpu/esimd_kernels/norm_gemv_norm_fp16.h:56-98)."""
    v = residual.float()
    n = v * torch.rsqrt(v.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (n * w1.float()).to(residual.dtype), (n * w2.float()).to(residual.dtype)
