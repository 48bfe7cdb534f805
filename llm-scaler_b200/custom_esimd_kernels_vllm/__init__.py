"""B200 (sm_100a) implementation of the quantized-linear / MoE-GEMM ops of intel/llm-scaler's
`custom_esimd_kernels_vllm` package, importable under the same name.

Importing the package loads libb2q.so (hand-written CUDA behind a C ABI, see include/b2q.h) and
registers the reference's torch custom-op schemas for the CUDA dispatch key.  There is no CPU path:
the import fails if the library is missing and every op rejects non-CUDA tensors.
"""
from . import _lib  # noqa: F401  (fails loudly when libb2q.so is absent)
from . import _register  # noqa: F401
from .ops import *  # noqa: F401,F403
from .ops import (  # noqa: F401
    esimd_gemv_fp8_pern, esimd_gemv_fp8_pern_fused2, esimd_gemv_fp8_pern_fused3, esimd_gemv_fp8_pert,
    esimd_gemv_fp8_pert_bmg, esimd_gemv_fp8_pert_fused2, esimd_gemv_fp8_pert_fused3, esimd_gemm_fp8_pert,
    esimd_gemm_fp8_blockscale, esimd_gemv_fp8_blockscale_fused2, esimd_gemv_int4, esimd_gemv_int4_fused2,
    esimd_gemm_int4_pgrp, esimd_moe_topk, esimd_moe_scatter, esimd_moe_scatter_fused, esimd_moe_silu_mul,
    esimd_moe_gather, esimd_moe_gemm_fp8, esimd_moe_gemm_fp8_pert, esimd_moe_gemm_fp8_blockscale, moe_topk_int4,
    to_cutlass_nmajor_int4, cutlass_nmajor_int4_to_signed, prepare_cutlass_nmajor_int4_weight, precompute_moe_route,
    moe_silu_mul_int4, moe_route_gather_int4, moe_gemm_int4_nmajor, moe_prefill_full_int4, moe_topk_softmax,
    esimd_resadd_norm_gemv_fp8_pert, esimd_resadd_norm_gemv_int4_pert, esimd_resadd_norm_gemv2_fp8_pert, q4_0_quantize,
    esimd_norm_gemv_fp8_pert, esimd_norm_gemv_fp8_blockscale, esimd_norm_gemv_int4_pert,
    moe_router_forward_int4, moe_router_topk_int4, moe_forward_full_int4, moe_shared_expert_forward_int4_nmajor,
    moe_forward_cutlass_nmajor_int4_full, esimd_scaled_resadd_norm_gemv_fp8_pert, esimd_norm_gemv_norm_fp16,
)

launch_count = _lib.launch_count
last_kernel = _lib.last_kernel
set_force_kernel = _lib.set_force_kernel
set_overlap_mode = _lib.set_overlap_mode
