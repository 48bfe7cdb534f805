"""Python wrappers with the names, argument order and docstring contracts of the reference package
(python/custom_esimd_kernels_vllm/ops.py).  Each is a one-line forward to the torch custom op, so a
caller can use either `custom_esimd_kernels_vllm.esimd_gemv_int4(...)` or
`torch.ops.custom_esimd_kernels_vllm.esimd_gemv_int4(...)`.

Differences from the reference surface, all widening: activations / outputs may be bf16 as well as
fp16; INT4 scales may be bf16 / fp16 / fp32; per-channel FP8 scales may be fp16 / bf16 / fp32; every
dense op accepts any M >= 1 (the reference caps its kernels at M = 1 / 64 / 128).  Device checks
test for "cuda" where the reference tests for "xpu".
"""
import torch
import torch.nn.functional as F

from . import _register  # noqa: F401  (defines the ops)
from . import _impl

_ops = torch.ops.custom_esimd_kernels_vllm
_prefill = torch.ops.moe_int4_prefill_ops
_moe_int4 = torch.ops.moe_int4_ops


# ---- FP8 GEMV / GEMM (ops.py:8-63, 91-143, 799-835 of the reference) ----
def esimd_gemv_fp8_pern(input, weight, weight_scale, output, N, K):
    """FP8 weight GEMV with one scale per output row.  input [M, K], weight [N, K] fp8, scale [N], output [M, N]."""
    return _ops.esimd_gemv_fp8_pern(input, weight, weight_scale, output, N, K)


def esimd_gemv_fp8_pern_fused2(input, w0, s0, o0, N0, w1, s1, o1, N1, K):
    return _ops.esimd_gemv_fp8_pern_fused2(input, w0, s0, o0, N0, w1, s1, o1, N1, K)


def esimd_gemv_fp8_pern_fused3(input, w0, s0, o0, N0, w1, s1, o1, N1, w2, s2, o2, N2, K):
    return _ops.esimd_gemv_fp8_pern_fused3(input, w0, s0, o0, N0, w1, s1, o1, N1, w2, s2, o2, N2, K)


def esimd_gemv_fp8_pert(input, weight, weight_scale, output):
    """FP8 weight GEMV with a per-tensor fp32 scalar scale read on the device."""
    return _ops.esimd_gemv_fp8_pert(input, weight, weight_scale, output)


def esimd_gemv_fp8_pert_bmg(input, weight, weight_scale, output):
    return _ops.esimd_gemv_fp8_pert_bmg(input, weight, weight_scale, output)


def esimd_gemv_fp8_pert_fused2(input, w0, s0, o0, w1, s1, o1):
    return _ops.esimd_gemv_fp8_pert_fused2(input, w0, s0, o0, w1, s1, o1)


def esimd_gemv_fp8_pert_fused3(input, w0, s0, o0, w1, s1, o1, w2, s2, o2):
    return _ops.esimd_gemv_fp8_pert_fused3(input, w0, s0, o0, w1, s1, o1, w2, s2, o2)


def esimd_gemm_fp8_pert(input, weight, weight_scale, output):
    """FP8 GEMM with per-tensor scale, any M."""
    return _ops.esimd_gemm_fp8_pert(input, weight, weight_scale, output)


def esimd_gemm_fp8_blockscale(input, weight, weight_scale, output, block_n=128, block_k=128):
    """FP8 128x128 block-scaled GEMM, w8a16: the activation is not quantised."""
    return _ops.esimd_gemm_fp8_blockscale(input, weight, weight_scale, output, block_n, block_k)


def esimd_gemv_fp8_blockscale_fused2(input, w0, s0, o0, w1, s1, o1, block_n=128, block_k=128):
    return _ops.esimd_gemv_fp8_blockscale_fused2(input, w0, s0, o0, w1, s1, o1, block_n, block_k)


# ---- INT4 (ops.py:146-207) ----
def esimd_gemv_int4(input, weight, weight_scale, output):
    """Symmetric INT4 (g=128) weight GEMV.  weight uint8 [N, K/2] (low nibble = even k), scale [N, K/128]."""
    return _ops.esimd_gemv_int4(input, weight, weight_scale, output)


def esimd_gemv_int4_fused2(input, w0, s0, o0, w1, s1, o1):
    return _ops.esimd_gemv_int4_fused2(input, w0, s0, o0, w1, s1, o1)


def esimd_gemm_int4_pgrp(input, weight, weight_scale, output):
    """INT4 GEMM with per-group scale for M >= 2 (no upper bound on M here)."""
    return _ops.esimd_gemm_int4_pgrp(input, weight, weight_scale, output)


# ---- MoE auxiliary ops + FP8 grouped GEMM (ops.py:633-859) ----
def esimd_moe_topk(router_logits, top_values, top_indices, T):
    return _ops.esimd_moe_topk(router_logits, top_values, top_indices, T)


def esimd_moe_scatter(hidden_states, router_top_value, sorted_token_ids, scattered_hidden, scattered_weights, K, topk,
                      total_expanded):
    return _ops.esimd_moe_scatter(hidden_states, router_top_value, sorted_token_ids, scattered_hidden,
                                  scattered_weights, K, topk, total_expanded)


def esimd_moe_scatter_fused(hidden_states, top_values, top_indices, scattered_hidden, scattered_weights, topk_ids,
                            expert_start, max_tokens_out, K, topk, T, num_experts):
    return _ops.esimd_moe_scatter_fused(hidden_states, top_values, top_indices, scattered_hidden, scattered_weights,
                                        topk_ids, expert_start, max_tokens_out, K, topk, T, num_experts)


def esimd_moe_silu_mul(input, output, N_gate_up, N_half, total_rows):
    return _ops.esimd_moe_silu_mul(input, output, N_gate_up, N_half, total_rows)


def esimd_moe_gather(moe_output, topk_ids, scattered_weights, final_hidden, K, topk, T):
    return _ops.esimd_moe_gather(moe_output, topk_ids, scattered_weights, final_hidden, K, topk, T)


def esimd_moe_gemm_fp8(input, weight, scale, output, expert_idx, N, K, num_experts, max_tokens_per_expert):
    """Grouped GEMM, FP8 E5M2 weights [E, N, K] with per-N fp32 scales [E, N]."""
    return _ops.esimd_moe_gemm_fp8(input, weight, scale, output, expert_idx, N, K, num_experts, max_tokens_per_expert)


def esimd_moe_gemm_fp8_pert(input, weight, scale, output, expert_idx, N, K, num_experts, max_tokens_per_expert):
    return _ops.esimd_moe_gemm_fp8_pert(input, weight, scale, output, expert_idx, N, K, num_experts,
                                        max_tokens_per_expert)


def esimd_moe_gemm_fp8_blockscale(input, weight, weight_scale, output, expert_idx, N, K, num_experts, block_n=128,
                                  block_k=128):
    return _ops.esimd_moe_gemm_fp8_blockscale(input, weight, weight_scale, output, expert_idx, N, K, num_experts,
                                              block_n, block_k)


# ---- INT4 MoE (ops.py:1233-1362) ----
def moe_topk_int4(logits, top_k, n_routed_experts, norm=True):
    return _moe_int4.moe_topk_int4(logits.contiguous(), top_k, n_routed_experts, norm)


def moe_router_forward_int4(x, weight, scale, use_ggml_layout=False):
    """INT4 router GEMV, logits [T, E] (ops.py:1139-1150)."""
    return _moe_int4.moe_router_forward_int4(x.contiguous(), weight, scale, use_ggml_layout)


def moe_router_topk_int4(x, weight, scale, use_ggml_layout, top_k, n_routed_experts, norm=True):
    """INT4 router followed by top-k (ops.py:1153-1168)."""
    return _moe_int4.moe_router_topk_int4(x.contiguous(), weight, scale, use_ggml_layout, top_k, n_routed_experts, norm)


def moe_forward_full_int4(x, logits, gate_up_qweight, gate_up_scales, shared_gate_up_weight, shared_gate_up_scale,
                          down_qweight, down_scales, shared_down_weight, shared_down_scale, shared_expert_gate_weight,
                          top_k, num_shared_experts, n_routed_experts, use_ggml_layout=False):
    """INT4 MoE decode pipeline with the shared expert: topk + up + down + finalize (ops.py:1171-1206)."""
    return _moe_int4.moe_forward_full_int4(x, logits, gate_up_qweight, gate_up_scales, shared_gate_up_weight,
                                           shared_gate_up_scale, down_qweight, down_scales, shared_down_weight,
                                           shared_down_scale, shared_expert_gate_weight, top_k, num_shared_experts,
                                           n_routed_experts, use_ggml_layout)


def moe_shared_expert_forward_int4_nmajor(x, gate_up_qweight, gate_up_scale, down_qweight, down_scale, gate_weight):
    """Sigmoid-gated shared expert with N-major uint8 INT4 weights (ops.py:1209-1230)."""
    return _moe_int4.moe_shared_expert_forward_int4_nmajor(x, gate_up_qweight, gate_up_scale, down_qweight,
                                                           down_scale, gate_weight)


def moe_forward_cutlass_nmajor_int4_full(x, logits, w13, w13_scales, w2, w2_scales, shared_gu_w, shared_d_w,
                                         shared_gate_w, top_k, num_shared_experts, n_routed_experts):
    """Decode pipeline on two's-complement N-major INT4 experts with a 16-bit shared expert (ops.py:1674-1690)."""
    return _moe_int4.moe_forward_cutlass_nmajor_int4_full(x, logits, w13, w13_scales, w2, w2_scales, shared_gu_w,
                                                          shared_d_w, shared_gate_w, top_k, num_shared_experts,
                                                          n_routed_experts)


def to_cutlass_nmajor_int4(qweight):
    """int32 [.., N, K/8] -> uint8 [.., N, K/2], low nibble = even k (pure torch, device agnostic)."""
    if qweight.dtype == torch.uint8:
        return qweight.contiguous()
    if qweight.dtype not in (torch.int32, torch.int64):
        raise TypeError(f"unsupported qweight dtype: {qweight.dtype}")
    if qweight.dim() not in (2, 3):
        raise ValueError(f"expected [N,K/8] or [E,N,K/8], got {tuple(qweight.shape)}")
    u = qweight.to(torch.int64) & 0xFFFFFFFF
    sh = torch.arange(8, device=qweight.device, dtype=torch.int64) * 4
    nib = ((u.unsqueeze(-1) >> sh) & 0xF).to(torch.uint8).reshape(*qweight.shape[:-1], qweight.shape[-1] * 8)
    return (nib[..., 0::2] | (nib[..., 1::2] << 4)).contiguous()


def cutlass_nmajor_int4_to_signed(qweight_u4):
    """uint4 bytes -> two's-complement int4 bytes (value - 8 per nibble); the pure-torch zero-point fold."""
    if qweight_u4.dtype != torch.uint8:
        raise TypeError(f"expected uint8 qweight, got {qweight_u4.dtype}")
    lo = ((qweight_u4 & 0xF).to(torch.int16) - 8) & 0xF
    hi = (((qweight_u4 >> 4) & 0xF).to(torch.int16) - 8) & 0xF
    return (lo | (hi << 4)).to(torch.uint8).contiguous()


def prepare_cutlass_nmajor_int4_weight(qweight):
    return cutlass_nmajor_int4_to_signed(to_cutlass_nmajor_int4(qweight))


def precompute_moe_route(topk_weights, topk_ids, num_experts):
    """Sort token routes by expert.  Returns sorted_rows (int64), sorted_weights, rows_per_expert (int32)."""
    if topk_weights.device.type == "cuda" and topk_ids.device.type == "cuda":
        return _moe_int4.moe_route_precompute_int4(topk_weights.contiguous(), topk_ids.contiguous(), num_experts)
    num_rows, top_k = topk_ids.shape
    flat_experts = topk_ids.reshape(-1).to(torch.int64)
    flat_rows = torch.arange(num_rows, device=topk_ids.device, dtype=torch.int64).repeat_interleave(top_k)
    order = torch.argsort(flat_experts, stable=True)
    rows_per_expert = torch.bincount(flat_experts[order], minlength=num_experts).to(torch.int32)
    return flat_rows[order].contiguous(), topk_weights.reshape(-1)[order].contiguous(), rows_per_expert.contiguous()


def moe_silu_mul_int4(gate_up):
    if gate_up.device.type == "cuda":
        return _moe_int4.moe_silu_mul_int4(gate_up.contiguous())
    inter = gate_up.shape[1] // 2
    return (F.silu(gate_up[:, :inter].float()) * gate_up[:, inter:].float()).to(gate_up.dtype).contiguous()


def moe_route_gather_int4(route_output, sorted_rows, sorted_weights, n_tokens):
    return _moe_int4.moe_route_gather_int4(route_output.contiguous(), sorted_rows.contiguous(),
                                           sorted_weights.contiguous(), n_tokens)


def moe_gemm_int4_nmajor(x, weight, scale, expert_idx, group_size=128):
    return _moe_int4.moe_gemm_int4_nmajor(x, weight, scale, expert_idx, group_size)


# ---- INT4 MoE prefill pipeline (csrc/moe_prefill/moe_prefill_int4.sycl:992-1013) ----
def moe_prefill_full_int4(x, router_logits, gate_up_weight, gate_up_scale, down_weight, down_scale, top_k,
                          n_routed_experts):
    return _prefill.moe_prefill_full_int4(x, router_logits, gate_up_weight, gate_up_scale, down_weight, down_scale,
                                          top_k, n_routed_experts)


def moe_topk_softmax(router_logits, top_k, num_experts):
    return _prefill.moe_topk_softmax(router_logits, top_k, num_experts)


# ---- additions that have no reference counterpart: activations quantised per token per 128 columns (W8A8) ----
act_quant_fp8_1x128 = _impl.act_quant_fp8_1x128
gemm_fp8_block_w8a8 = _impl.gemm_fp8_block_w8a8
dequant_int4 = _impl.dequant_int4
dequant_fp8 = _impl.dequant_fp8


# ---- residual add + RMSNorm + decode GEMV (reference ops.py:411-489) and the load-time Q4_0 quantiser ----
def esimd_resadd_norm_gemv_fp8_pert(hidden_states, residual, norm_weight, gemv_weight, gemv_scale, output, normed_out, eps):
    """residual += hidden_states (in place); normed_out = rmsnorm(residual) * norm_weight;
    output = normed_out @ dequant(gemv_weight)^T with a per-tensor fp32 scale.  Returns output."""
    return _ops.esimd_resadd_norm_gemv_fp8_pert(hidden_states, residual, norm_weight, gemv_weight, gemv_scale, output, normed_out, eps)


def esimd_resadd_norm_gemv_int4_pert(hidden_states, residual, norm_weight, gemv_weight, gemv_scale, output, normed_out, eps):
    """As esimd_resadd_norm_gemv_fp8_pert with INT4 g=128 weights (int32 [N, K/8], scales [N, K/128])."""
    return _ops.esimd_resadd_norm_gemv_int4_pert(hidden_states, residual, norm_weight, gemv_weight, gemv_scale, output, normed_out, eps)


def esimd_resadd_norm_gemv2_fp8_pert(hidden_states, residual, norm_weight, w0, s0, o0, w1, s1, o1, eps):
    """Residual add + RMSNorm feeding two per-tensor FP8 GEMVs (o0, o1).  Returns o0."""
    return _ops.esimd_resadd_norm_gemv2_fp8_pert(hidden_states, residual, norm_weight, w0, s0, o0, w1, s1, o1, eps)


def esimd_scaled_resadd_norm_gemv_fp8_pert(hidden_states, residual, norm_weight, qkv_weight, qkv_scale, qkv_out, eps,
                                           scalar):
    """residual <- (hidden + residual) * scalar; qkv_out = FP8 GEMV of rmsnorm(residual) * norm_weight (ops.py:1832-1849)."""
    return _ops.esimd_scaled_resadd_norm_gemv_fp8_pert(hidden_states, residual, norm_weight, qkv_weight, qkv_scale,
                                                       qkv_out, eps, scalar)


def esimd_norm_gemv_norm_fp16(residual, scale_with_root, proj_w, pre_ff_w, router_logits, moe_input, eps):
    """router_logits = (rmsnorm(residual) * scale_with_root) @ proj_w^T and moe_input = rmsnorm(residual) * pre_ff_w from
    one shared 1/rms (ops.py:1801-1829)."""
    return _ops.esimd_norm_gemv_norm_fp16(residual, scale_with_root, proj_w, pre_ff_w, router_logits, moe_input, eps)


def q4_0_quantize(input, out_qweight, out_scale):
    """GGML Q4_0 (group 128) on the device: fills out_qweight int32 [M, K/8] and out_scale fp16 [M, K/128]."""
    _ops.q4_0_quantize(input, out_qweight, out_scale)


def esimd_norm_gemv_fp8_pert(x, z, norm_weight, gemv_weight, gemv_scale, output, HV, V, eps):
    """output[1, N] = (rmsnorm(x) * norm_weight * silu(z)).flatten() @ dequant(gemv_weight)^T, per-tensor FP8 scale."""
    return _ops.esimd_norm_gemv_fp8_pert(x, z, norm_weight, gemv_weight, gemv_scale, output, HV, V, eps)


def esimd_norm_gemv_fp8_blockscale(x, z, norm_weight, gemv_weight, gemv_scale, output, HV, V, eps):
    """As esimd_norm_gemv_fp8_pert with 128 x 128 block scales."""
    return _ops.esimd_norm_gemv_fp8_blockscale(x, z, norm_weight, gemv_weight, gemv_scale, output, HV, V, eps)


def esimd_norm_gemv_int4_pert(x, z, norm_weight, gemv_weight, gemv_scale, output, HV, V, eps):
    """As esimd_norm_gemv_fp8_pert with INT4 g=128 weights."""
    return _ops.esimd_norm_gemv_int4_pert(x, z, norm_weight, gemv_weight, gemv_scale, output, HV, V, eps)


# ---- GELU-tanh activation and the block-FP8 + 16-bit dual GEMV (ops.py:117-128, :718-726 of the reference) ----
def esimd_moe_gelu_tanh_mul(input, output, N_gate_up, N_half, total_rows):
    """GELU_tanh(gate) * up over [rows, 2 * N_half] -> [rows, N_half]."""
    return _ops.esimd_moe_gelu_tanh_mul(input, output, N_gate_up, N_half, total_rows)


def esimd_gemv_fp8_blockscale_fp16_fused2(input, w0, s0, o0, w1, o1, block_n=128, block_k=128):
    """Block-scaled e4m3 w0 and dense 16-bit w1 applied to the same input; results in o0 / o1, returns o0."""
    return _ops.esimd_gemv_fp8_blockscale_fp16_fused2(input, w0, s0, o0, w1, o1, block_n, block_k)


# ---- moe_ops: FP8 (e4m3, one fp32 scale per expert) MoE with GELU-tanh (ops.py:1693-1790 of the reference) ----
_moe_batch = torch.ops.moe_ops


class _MoeOpsNamespace:
    """`custom_esimd_kernels_vllm.moe_ops.<op>`: the attribute callers of the reference use
    (vllm/patches/vllm_for_multi_arc.patch:3168); every name forwards to torch.ops.moe_ops."""

    def __getattr__(self, name):
        return getattr(_moe_batch, name)


moe_ops = _MoeOpsNamespace()


def moe_forward_full_fp8_grouped(x, gate_up_weight, gate_up_scale, down_weight, down_scale, routing_weights,
                                 expert_offsets, expert_tokens, top_k, n_routed_experts):
    return _moe_batch.moe_forward_full_fp8_grouped(x, gate_up_weight, gate_up_scale, down_weight, down_scale,
                                                   routing_weights, expert_offsets, expert_tokens, top_k, n_routed_experts)


def moe_forward_full_gelu_tanh(x, logits, gate_up_weight, gate_up_scale, down_weight, down_scale, top_k, n_routed_experts):
    return _moe_batch.moe_forward_full_gelu_tanh(x, logits, gate_up_weight, gate_up_scale, down_weight, down_scale,
                                                 top_k, n_routed_experts)


def moe_forward_full_gelu_tanh_routed(x, topk_weights, topk_indices, gate_up_weight, gate_up_scale, down_weight,
                                      down_scale, top_k, n_routed_experts):
    return _moe_batch.moe_forward_full_gelu_tanh_routed(x, topk_weights, topk_indices, gate_up_weight, gate_up_scale,
                                                        down_weight, down_scale, top_k, n_routed_experts)


def moe_forward_full_gelu_tanh_routed_decode(x, topk_weights, topk_indices, gate_up_weight, gate_up_scale, down_weight,
                                             down_scale, top_k, n_routed_experts):
    return _moe_batch.moe_forward_full_gelu_tanh_routed_decode(x, topk_weights, topk_indices, gate_up_weight,
                                                               gate_up_scale, down_weight, down_scale, top_k,
                                                               n_routed_experts)


def moe_forward_full_gelu_tanh_routed_no_accum(x, topk_weights, topk_indices, gate_up_weight, gate_up_scale, down_weight,
                                               down_scale, top_k, n_routed_experts):
    return _moe_batch.moe_forward_full_gelu_tanh_routed_no_accum(x, topk_weights, topk_indices, gate_up_weight,
                                                                 gate_up_scale, down_weight, down_scale, top_k,
                                                                 n_routed_experts)


def moe_forward_full_gelu_tanh_decode(x, logits, gate_up_weight, gate_up_scale, down_weight, down_scale,
                                      per_expert_scale, top_k, n_routed_experts):
    return _moe_batch.moe_forward_full_gelu_tanh_decode(x, logits, gate_up_weight, gate_up_scale, down_weight,
                                                        down_scale, per_expert_scale, top_k, n_routed_experts)
