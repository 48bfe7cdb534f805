"""Registers the reference's torch custom ops for the CUDA dispatch key.

Schema strings are copied character for character from the reference registration units
(csrc/xpu/torch_extension.cc, torch_extension_gemm.cc, torch_extension_moe.cc,
torch_extension_topk_v2.cc, csrc/moe_prefill/moe_prefill_int4.sycl:992-1013,
csrc/moe_batch/moe_int4.sycl:3896-3937) so that callers written against
`torch.ops.custom_esimd_kernels_vllm.*`, `torch.ops.moe_int4_prefill_ops.*`,
`torch.ops.moe_int4_ops.*` and `torch.ops.esimd_topk_v2.*` run unchanged.  The reference
registers them for the XPU key; here the implementation key is CUDA.  Dense ops keep the
reference's alias-return convention: the caller pre-allocates `output` and gets it back.
"""
import ctypes
import os

import torch

from . import _impl as I
from . import _lib as L

_LIBS = {}
IMPLEMENTED = {}      # namespace -> names of the ops registered with an implementation

# The dense linears are implemented for the CUDA key in C++ (csrc/torch_ops.cpp -> libb2q_torch.so, straight over the
# C ABI): loading that library registers them, and the Python implementations below are then not attached to those
# names.  B2Q_PYTHON_DISPATCH=1 keeps every op on its Python implementation (the two must agree; a test runs both).
CPP_OPS = frozenset()
_CPP_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libb2q_torch.so")
# B2Q_CHECK_STATUS=1 (debugging, tests): every op synchronises after its launches and raises if a bounded device-side
# wait has expired, instead of leaving that to a caller who polls b2q_device_status.  It implies Python dispatch.
CHECK_STATUS = os.environ.get("B2Q_CHECK_STATUS") == "1"
if os.environ.get("B2Q_PYTHON_DISPATCH") != "1" and not CHECK_STATUS:
    if not os.path.exists(_CPP_PATH):
        raise ImportError("b2q: %s is missing; build it with `python llm-scaler_b200/build.py`" % _CPP_PATH)
    torch.ops.load_library(_CPP_PATH)
    _h = ctypes.CDLL(_CPP_PATH)
    _h.b2q_torch_ops.restype = ctypes.c_char_p
    CPP_OPS = frozenset(_h.b2q_torch_ops().decode().split(","))


def _lib(ns):
    if ns not in _LIBS:
        _LIBS[ns] = torch.library.Library(ns, "DEF")
    return _LIBS[ns]


def _checked(fn, what):
    def run(*a, **k):
        out = fn(*a, **k)
        code = L.device_status()
        if code:
            raise RuntimeError("b2q: %s: a bounded device-side wait expired (code %d); results are not valid" % (what, code))
        return out
    return run


def _op(ns, schema, fn, meta=None):
    lib = _lib(ns)
    lib.define(schema)
    name = schema.split("(", 1)[0]
    IMPLEMENTED.setdefault(ns, []).append(name)
    if CHECK_STATUS:
        fn = _checked(fn, ns + "::" + name)
    if not (ns == "custom_esimd_kernels_vllm" and name in CPP_OPS):
        lib.impl(name, fn, "CUDA")
    if meta is not None:
        lib.impl(name, meta, "Meta")


NS = "custom_esimd_kernels_vllm"


# ---------------------------------------------------------------- dense INT4
def _gemv_int4(input, weight, weight_scale, output):
    return I.linear_int4(input, weight, weight_scale, output)


def _gemv_int4_fused2(input, w0, s0, o0, w1, s1, o1):
    I.linear_int4(input, w0, s0, o0)
    I.linear_int4(input, w1, s1, o1)
    return o0


_op(NS, "esimd_gemv_int4(Tensor input, Tensor weight, Tensor weight_scale, Tensor output) -> Tensor",
    _gemv_int4, lambda i, w, s, o: o)
_op(NS, "esimd_gemv_int4_fused2(Tensor input, Tensor w0, Tensor s0, Tensor o0, Tensor w1, Tensor s1, Tensor o1) -> Tensor",
    _gemv_int4_fused2, lambda i, w0, s0, o0, w1, s1, o1: o0)
_op(NS, "esimd_gemm_int4_pgrp(Tensor input, Tensor weight, Tensor weight_scale, Tensor output) -> Tensor",
    _gemv_int4, lambda i, w, s, o: o)


# ---------------------------------------------------------------- dense FP8
def _fp8_pern(input, weight, weight_scale, output, N, K):
    return I.linear_fp8(input, weight, weight_scale, output, L.SCALE_CHANNEL, N, K)


def _fp8_pern_fused2(input, w0, s0, o0, N0, w1, s1, o1, N1, K):
    _fp8_pern(input, w0, s0, o0, N0, K)
    _fp8_pern(input, w1, s1, o1, N1, K)
    return o0


def _fp8_pern_fused3(input, w0, s0, o0, N0, w1, s1, o1, N1, w2, s2, o2, N2, K):
    _fp8_pern(input, w0, s0, o0, N0, K)
    _fp8_pern(input, w1, s1, o1, N1, K)
    _fp8_pern(input, w2, s2, o2, N2, K)
    return o0


def _fp8_pert(input, weight, weight_scale, output):
    return I.linear_fp8(input, weight, weight_scale, output, L.SCALE_TENSOR)


def _fp8_pert_fused2(input, w0, s0, o0, w1, s1, o1):
    _fp8_pert(input, w0, s0, o0)
    _fp8_pert(input, w1, s1, o1)
    return o0


def _fp8_pert_fused3(input, w0, s0, o0, w1, s1, o1, w2, s2, o2):
    _fp8_pert(input, w0, s0, o0)
    _fp8_pert(input, w1, s1, o1)
    _fp8_pert(input, w2, s2, o2)
    return o0


def _fp8_block(input, weight, weight_scale, output, block_n, block_k):
    I._chk(block_n == 128 and block_k == 128, "only block_n == block_k == 128 is supported")
    return I.linear_fp8(input, weight, weight_scale, output, L.SCALE_BLOCK128)


def _fp8_block_fused2(input, w0, s0, o0, w1, s1, o1, block_n, block_k):
    _fp8_block(input, w0, s0, o0, block_n, block_k)
    _fp8_block(input, w1, s1, o1, block_n, block_k)
    return o0


_op(NS, "esimd_gemv_fp8_pern(Tensor input, Tensor weight, Tensor weight_scale, Tensor output, int N, int K) -> Tensor",
    _fp8_pern, lambda i, w, s, o, N, K: o)
_op(NS, "esimd_gemv_fp8_pern_fused2(Tensor input, Tensor w0, Tensor s0, Tensor o0, int N0, "
        "Tensor w1, Tensor s1, Tensor o1, int N1, int K) -> Tensor", _fp8_pern_fused2)
_op(NS, "esimd_gemv_fp8_pern_fused3(Tensor input, Tensor w0, Tensor s0, Tensor o0, int N0, "
        "Tensor w1, Tensor s1, Tensor o1, int N1, Tensor w2, Tensor s2, Tensor o2, int N2, int K) -> Tensor",
    _fp8_pern_fused3)
_op(NS, "esimd_gemv_fp8_pert(Tensor input, Tensor weight, Tensor weight_scale, Tensor output) -> Tensor",
    _fp8_pert, lambda i, w, s, o: o)
_op(NS, "esimd_gemv_fp8_pert_bmg(Tensor input, Tensor weight, Tensor weight_scale, Tensor output) -> Tensor",
    _fp8_pert, lambda i, w, s, o: o)
_op(NS, "esimd_gemv_fp8_pert_fused2(Tensor input, Tensor w0, Tensor s0, Tensor o0, Tensor w1, Tensor s1, Tensor o1) -> Tensor",
    _fp8_pert_fused2)
_op(NS, "esimd_gemv_fp8_pert_fused3(Tensor input, Tensor w0, Tensor s0, Tensor o0, Tensor w1, Tensor s1, Tensor o1, "
        "Tensor w2, Tensor s2, Tensor o2) -> Tensor", _fp8_pert_fused3)
_op(NS, "esimd_gemm_fp8_pert(Tensor input, Tensor weight, Tensor weight_scale, Tensor output) -> Tensor",
    _fp8_pert, lambda i, w, s, o: o)
_op(NS, "esimd_gemm_fp8_blockscale(Tensor input, Tensor weight, Tensor weight_scale, Tensor output, int block_n, int block_k) -> Tensor",
    _fp8_block, lambda i, w, s, o, bn, bk: o)
_op(NS, "esimd_gemv_fp8_blockscale_fused2(Tensor input, Tensor w0, Tensor s0, Tensor(a!) o0, Tensor w1, Tensor s1, "
        "Tensor(b!) o1, int block_n, int block_k) -> Tensor(a!)", _fp8_block_fused2)


# ---------------------------------------------------------------- MoE aux + FP8 grouped GEMM
def _moe_topk(router_logits, top_values, top_indices, T):
    I._chk(router_logits.shape[0] >= T, "T exceeds router_logits rows")
    I.moe_topk(router_logits[:T], top_values.shape[1], True, top_values, top_indices)
    return top_values


def _moe_scatter_fused(hidden_states, top_values, top_indices, scattered_hidden, scattered_weights, topk_ids,
                       expert_start, max_tokens_out, K, topk, T, num_experts):
    ids = top_indices[:T].contiguous()
    offsets, tokens, p2p, rows = I.moe_route(ids, num_experts)
    n = T * topk
    gathered = I.gather_rows(hidden_states[:T].contiguous(), tokens, topk, n)
    scattered_hidden[:n].copy_(gathered)
    scattered_weights[:n].copy_(top_values[:T].reshape(-1)[tokens.long()])
    topk_ids.reshape(-1)[:n].copy_(p2p)
    expert_start.view(torch.int32)[: num_experts + 1].copy_(offsets)
    max_tokens_out.copy_(rows.max().reshape(1))
    return scattered_hidden


def _moe_scatter(hidden_states, router_top_value, sorted_token_ids, scattered_hidden, scattered_weights, K, topk,
                 total_expanded):
    ids = sorted_token_ids[:total_expanded].contiguous()
    scattered_hidden[:total_expanded].copy_(I.gather_rows(hidden_states.contiguous(), ids, topk, total_expanded))
    scattered_weights[:total_expanded].copy_(router_top_value.reshape(-1)[ids.long()])
    return scattered_hidden


def _moe_silu_mul(input, output, N_gate_up, N_half, total_rows):
    I._chk(N_gate_up == 2 * N_half, "N_gate_up must be 2 * N_half")
    I.silu_mul(input[:total_rows], output[:total_rows])
    return output


def _moe_gather(moe_output, topk_ids, scattered_weights, final_hidden, K, topk, T):
    I.moe_combine(moe_output, scattered_weights, topk_ids.reshape(-1).contiguous(), T, topk, final_hidden, w_by_row=True)
    return final_hidden


def _moe_gemm_fp8_mode(mode):
    def fn(input, weight, scale, output, expert_idx, N, K, num_experts, max_tokens_per_expert):
        w = weight if weight.dtype != torch.uint8 else weight.view(torch.float8_e5m2)
        I.moe_gemm_fp8(input, w.reshape(num_experts, N, K), scale, expert_idx, input.shape[0], mode, out=output)
        return output
    return fn


def _moe_gemm_fp8_block(input, weight, weight_scale, output, expert_idx, N, K, num_experts, block_n, block_k):
    I._chk(block_n == 128 and block_k == 128, "only 128x128 blocks are supported")
    I.moe_gemm_fp8(input, weight.reshape(num_experts, N, K), weight_scale, expert_idx, input.shape[0],
                   L.SCALE_BLOCK128, out=output)
    return output


_op(NS, "esimd_moe_topk(Tensor router_logits, Tensor top_values, Tensor top_indices, int T) -> Tensor", _moe_topk)
_op(NS, "esimd_moe_scatter(Tensor hidden_states, Tensor router_top_value, Tensor sorted_token_ids, "
        "Tensor scattered_hidden, Tensor scattered_weights, int K, int topk, int total_expanded) -> Tensor", _moe_scatter)
_op(NS, "esimd_moe_scatter_fused(Tensor hidden_states, Tensor top_values, Tensor top_indices, "
        "Tensor scattered_hidden, Tensor scattered_weights, Tensor topk_ids, Tensor expert_start, Tensor max_tokens_out, "
        "int K, int topk, int T, int num_experts) -> Tensor", _moe_scatter_fused)
# residual add + RMSNorm + decode GEMV (reference: ops.py:411-489; kernels esimd_kernels/resadd_norm_gemv_int4.h,
# norm_gemv_fused.h).  FP8 with one GEMV: the norm runs inside the GEMV's activation pre-pass (two launches in all).
# INT4 and the two-GEMV form: one norm kernel, then the ordinary GEMV(s) on normed_out; the kernels overlap on the stream.
def _resadd_norm_gemv_fp8_pert(hidden_states, residual, norm_weight, gemv_weight, gemv_scale, output, normed_out, eps):
    _chk_scale = I._chk(gemv_scale.numel() == 1 and gemv_scale.dtype == torch.float32, "per-tensor scale must be one fp32")
    return I.resadd_norm_linear_fp8(hidden_states, residual, norm_weight, normed_out, eps, 1.0, gemv_weight, gemv_scale,
                                    output, L.SCALE_TENSOR)


def _resadd_norm_gemv_int4_pert(hidden_states, residual, norm_weight, gemv_weight, gemv_scale, output, normed_out, eps):
    I.resadd_rmsnorm(hidden_states, residual, norm_weight, normed_out, eps)
    return I.linear_int4(normed_out, gemv_weight, gemv_scale, output)


def _resadd_norm_gemv2_fp8_pert(hidden_states, residual, norm_weight, w0, s0, o0, w1, s1, o1, eps):
    normed = torch.empty_like(hidden_states)
    I.resadd_rmsnorm(hidden_states, residual, norm_weight, normed, eps)
    I.linear_fp8(normed, w0, s0, o0, L.SCALE_TENSOR)
    I.linear_fp8(normed, w1, s1, o1, L.SCALE_TENSOR)
    return o0


def _scaled_resadd_norm_gemv_fp8_pert(hidden_states, residual, norm_weight, qkv_weight, qkv_scale, qkv_out, eps, scalar):
    normed = torch.empty_like(residual)
    I.resadd_norm_linear_fp8(hidden_states, residual, norm_weight, normed, eps, scalar, qkv_weight, qkv_scale, qkv_out,
                             L.SCALE_TENSOR)


def _norm_gemv_norm_fp16(residual, scale_with_root, proj_w, pre_ff_w, router_logits, moe_input, eps):
    # shared 1/rms, two post-norm scales in one launch; the 16-bit dense router projection is a plain library GEMM
    router_in = torch.empty_like(residual)
    I.rmsnorm_fused(None, residual, 1.0, scale_with_root, router_in, pre_ff_w, moe_input, eps)
    torch.matmul(router_in, proj_w.t(), out=router_logits)


_op(NS, "esimd_scaled_resadd_norm_gemv_fp8_pert(Tensor hidden_states, Tensor residual, "
        "Tensor norm_weight, Tensor qkv_weight, Tensor qkv_scale, Tensor qkv_out, "
        "float eps, float scalar) -> ()", _scaled_resadd_norm_gemv_fp8_pert)
_op(NS, "esimd_norm_gemv_norm_fp16(Tensor residual, Tensor scale_with_root, "
        "Tensor proj_w, Tensor pre_ff_w, Tensor router_logits, Tensor moe_input, "
        "float eps) -> ()", _norm_gemv_norm_fp16)
_op(NS, "esimd_resadd_norm_gemv_fp8_pert(Tensor hidden_states, Tensor residual, Tensor norm_weight, Tensor gemv_weight, "
        "Tensor gemv_scale, Tensor output, Tensor normed_out, float eps) -> Tensor", _resadd_norm_gemv_fp8_pert)
_op(NS, "esimd_resadd_norm_gemv_int4_pert(Tensor hidden_states, Tensor residual, Tensor norm_weight, Tensor gemv_weight, "
        "Tensor gemv_scale, Tensor output, Tensor normed_out, float eps) -> Tensor", _resadd_norm_gemv_int4_pert)
_op(NS, "esimd_resadd_norm_gemv2_fp8_pert(Tensor hidden_states, Tensor residual, Tensor norm_weight, Tensor w0, Tensor s0, "
        "Tensor o0, Tensor w1, Tensor s1, Tensor o1, float eps) -> Tensor", _resadd_norm_gemv2_fp8_pert)

# gated RMSNorm + decode GEMV (reference: ops.py:492-565, torch_extension.cc:117-121)
def _norm_gemv(mode):
    def fn(x, z, norm_weight, gemv_weight, gemv_scale, output, HV, V, eps):
        if tuple(x.shape) != (HV, V):
            raise RuntimeError("b2q: x must be [HV, V]")
        normed = I.gated_rmsnorm(x, z, norm_weight, eps)
        if mode == "int4":
            return I.linear_int4(normed, gemv_weight, gemv_scale, output)
        return I.linear_fp8(normed, gemv_weight, gemv_scale, output, mode)
    return fn


_NORM_GEMV = "(Tensor x, Tensor z, Tensor norm_weight, Tensor gemv_weight, Tensor gemv_scale, Tensor output, int HV, int V, float eps) -> Tensor"
_op(NS, "esimd_norm_gemv_fp8_pert" + _NORM_GEMV, _norm_gemv(L.SCALE_TENSOR))
_op(NS, "esimd_norm_gemv_fp8_blockscale" + _NORM_GEMV, _norm_gemv(L.SCALE_BLOCK128))
_op(NS, "esimd_norm_gemv_int4_pert" + _NORM_GEMV, _norm_gemv("int4"))

# load-time quantiser (reference: csrc/xpu/torch_extension_q4_0.cc:78-83, module q4_0_quant_ops)
def _q4_0_quantize(input, out_qweight, out_scale):
    I.q4_0_quantize(input, out_qweight, out_scale)


_op(NS, "q4_0_quantize(Tensor input, Tensor(a!) out_qweight, Tensor(b!) out_scale) -> ()", _q4_0_quantize)
_op(NS, "esimd_moe_silu_mul(Tensor input, Tensor output, int N_gate_up, int N_half, int total_rows) -> Tensor", _moe_silu_mul)
_op(NS, "esimd_moe_gather(Tensor moe_output, Tensor topk_ids, Tensor scattered_weights, Tensor final_hidden, "
        "int K, int topk, int T) -> Tensor", _moe_gather)
_op(NS, "esimd_moe_gemm_fp8(Tensor input, Tensor weight, Tensor scale, Tensor output, Tensor expert_idx, "
        "int N, int K, int num_experts, int max_tokens_per_expert) -> Tensor", _moe_gemm_fp8_mode(L.SCALE_CHANNEL))
_op(NS, "esimd_moe_gemm_fp8_pert(Tensor input, Tensor weight, Tensor scale, Tensor output, Tensor expert_idx, "
        "int N, int K, int num_experts, int max_tokens_per_expert) -> Tensor", _moe_gemm_fp8_mode(L.SCALE_TENSOR))
_op(NS, "esimd_moe_gemm_fp8_blockscale(Tensor input, Tensor weight, Tensor weight_scale, Tensor(a!) output, "
        "Tensor expert_idx, int N, int K, int num_experts, int block_n, int block_k) -> Tensor(a!)", _moe_gemm_fp8_block)


def _topk_v2(router_logits, top_values, top_indices, T, num_experts, topk):
    I.moe_topk(router_logits[:T], topk, True, top_values, top_indices)
    return top_values


_op("esimd_topk_v2", "topk_v2(Tensor router_logits, Tensor top_values, Tensor top_indices, int T, int num_experts, int topk) -> Tensor",
    _topk_v2)


# ---------------------------------------------------------------- INT4 MoE prefill pipeline
PNS = "moe_int4_prefill_ops"


def _offsets_e1(expert_offsets, total):
    """The reference passes expert_offsets with E entries; the grouped GEMM wants the closing E+1-th."""
    tail = torch.full((1,), total, dtype=torch.int32, device=expert_offsets.device)
    return torch.cat([expert_offsets.to(torch.int32), tail])


def _prefill_topk_softmax(router_logits, top_k, num_experts):
    w, ids = I.moe_topk(router_logits.contiguous(), top_k, True)
    return [w, ids]


def _prefill_gather(selected_experts, num_experts):
    I._chk(selected_experts.dim() == 2 and selected_experts.dtype == torch.int32, "selected_experts must be int32 [T, k]")
    offsets, tokens, p2p, rows = I.moe_route(selected_experts.contiguous(), num_experts)
    return [offsets[:num_experts], tokens, p2p, rows]


def _prefill_up(x, gate_up_weight, gate_up_scale, expert_offsets, expert_tokens, top_k):
    total = expert_tokens.numel()
    off = _offsets_e1(expert_offsets, total)
    # result rows are indexed by pair (token * top_k + slot), as the reference's up kernel writes them
    return I.moe_gemm_int4(x, gate_up_weight, gate_up_scale, off, total, row_map=expert_tokens, row_div=top_k,
                           out_map=expert_tokens, act=L.ACT_SILU_MUL)


def _prefill_down(intermediate, down_weight, down_scale, expert_offsets, expert_tokens):
    total = expert_tokens.numel()
    off = _offsets_e1(expert_offsets, total)
    return I.moe_gemm_int4(intermediate, down_weight, down_scale, off, total, row_map=expert_tokens, row_div=1,
                           out_map=expert_tokens)


def _prefill_accumulate(output, routing_weights):
    T, k = routing_weights.shape
    return I.moe_combine(output.contiguous(), routing_weights.contiguous(), None, T, k)


def _prefill_accumulate_permuted(output_perm, routing_weights, pair_to_perm):
    T, k = routing_weights.shape
    return I.moe_combine(output_perm.contiguous(), routing_weights.contiguous(), pair_to_perm.contiguous(), T, k)


def _prefill_silu_mul(gate_up):
    return I.silu_mul(gate_up.contiguous())


def _prefill_scatter_x(x, expert_tokens, top_k):
    return I.gather_rows(x.contiguous(), expert_tokens.contiguous(), top_k)


def _prefill_full(x, router_logits, gate_up_weight, gate_up_scale, down_weight, down_scale, top_k, n_routed_experts):
    return I.moe_forward_int4(x, router_logits.contiguous(), gate_up_weight, gate_up_scale, down_weight, down_scale,
                              top_k, n_routed_experts)


_op(PNS, "moe_prefill_full_int4(Tensor x, Tensor router_logits, Tensor gate_up_weight, Tensor gate_up_scale, "
         "Tensor down_weight, Tensor down_scale, int top_k, int n_routed_experts) -> Tensor", _prefill_full)
_op(PNS, "moe_prefill_gather_forward_v2(Tensor selected_experts, int num_experts) -> Tensor[]", _prefill_gather)
_op(PNS, "moe_prefill_up_forward_v2(Tensor x, Tensor gate_up_weight, Tensor gate_up_scale, Tensor expert_offsets, "
         "Tensor expert_tokens, int top_k) -> Tensor", _prefill_up)
_op(PNS, "moe_prefill_down_forward_v2(Tensor intermediate, Tensor down_weight, Tensor down_scale, "
         "Tensor expert_offsets, Tensor expert_tokens) -> Tensor", _prefill_down)
_op(PNS, "moe_prefill_accumulate_forward_v2(Tensor output, Tensor routing_weights) -> Tensor", _prefill_accumulate)
_op(PNS, "moe_prefill_accumulate_permuted_forward_v2(Tensor output_perm, Tensor routing_weights, Tensor pair_to_perm) -> Tensor",
    _prefill_accumulate_permuted)
_op(PNS, "moe_prefill_silu_mul_forward(Tensor gate_up) -> Tensor", _prefill_silu_mul)
_op(PNS, "moe_prefill_scatter_x_forward(Tensor x, Tensor expert_tokens, int top_k) -> Tensor", _prefill_scatter_x)
_op(PNS, "moe_topk_softmax(Tensor router_logits, int top_k, int num_experts) -> Tensor[]", _prefill_topk_softmax)


# ---------------------------------------------------------------- moe_int4_ops (routed pieces)
INS = "moe_int4_ops"


def _topk_int4(logits, top_k, n_routed_experts, norm):
    return I.moe_topk(logits.contiguous(), top_k, bool(norm))


def _route_precompute(topk_weight, topk_idx, num_experts):
    ids = topk_idx.to(torch.int32).contiguous()
    offsets, tokens, p2p, rows = I.moe_route(ids, num_experts)
    top_k = ids.shape[1]
    sorted_rows = (tokens // top_k).to(torch.int64)
    sorted_weights = topk_weight.reshape(-1)[tokens.long()].contiguous()
    return sorted_rows, sorted_weights, rows


def _silu_mul_int4(gate_up):
    return I.silu_mul(gate_up.contiguous())


def _route_gather(route_output, sorted_rows, sorted_weights, n_tokens):
    total = sorted_rows.numel()
    I._chk(n_tokens > 0 and total % n_tokens == 0, "every token must own the same number of routed rows")
    k = total // n_tokens
    perm = torch.argsort(sorted_rows, stable=True).to(torch.int32).contiguous()
    return I.moe_combine(route_output.contiguous(), sorted_weights.contiguous(), perm, n_tokens, k, w_by_row=True)


def _gemm_int4_nmajor(x, weight, scale, expert_idx, group_size):
    I._chk(group_size == 128, "group_size must be 128")
    return I.moe_gemm_int4(x.contiguous(), weight, scale, expert_idx.to(torch.int32), x.shape[0])


_op(INS, "moe_topk_int4(Tensor logits, int top_k, int n_routed_experts, bool norm) -> (Tensor, Tensor)", _topk_int4)
_op(INS, "moe_route_precompute_int4(Tensor topk_weight, Tensor topk_idx, int num_experts) -> (Tensor, Tensor, Tensor)",
    _route_precompute)
_op(INS, "moe_silu_mul_int4(Tensor gate_up) -> Tensor", _silu_mul_int4)
_op(INS, "moe_route_gather_int4(Tensor route_output, Tensor sorted_rows, Tensor sorted_weights, int n_tokens) -> Tensor",
    _route_gather)
_op(INS, "moe_gemm_int4_nmajor(Tensor x, Tensor weight, Tensor scale, Tensor expert_idx, int group_size) -> Tensor",
    _gemm_int4_nmajor)



def _router_topk_int4(x, weight, scale, use_ggml_layout, top_k, n_routed_experts, norm):
    logits = I.moe_router_forward_int4(x, weight, scale, use_ggml_layout)
    return _topk_int4(logits, top_k, n_routed_experts, norm)


_op(INS, "moe_router_forward_int4(Tensor x, Tensor weight, Tensor scale, bool use_ggml_layout) -> Tensor",
    I.moe_router_forward_int4)
_op(INS, "moe_router_topk_int4(Tensor x, Tensor weight, Tensor scale, bool use_ggml_layout, int top_k, "
    "int n_routed_experts, bool norm) -> (Tensor, Tensor)", _router_topk_int4)
_op(INS, "moe_forward_full_int4(Tensor x, Tensor logits, "
    "Tensor gate_up_qweight, Tensor gate_up_scales, "
    "Tensor shared_gate_up_weight, Tensor shared_gate_up_scale, "
    "Tensor down_qweight, Tensor down_scales, "
    "Tensor shared_down_weight, Tensor shared_down_scale, "
    "Tensor shared_expert_gate_weight, "
    "int top_k, int num_shared_experts, int n_routed_experts, "
    "bool use_ggml_layout) -> Tensor", I.moe_forward_full_int4)
_op(INS, "moe_shared_expert_forward_int4_nmajor(Tensor x, "
    "Tensor gate_up_qweight, Tensor gate_up_scale, "
    "Tensor down_qweight, Tensor down_scale, "
    "Tensor gate_weight) -> Tensor", I.moe_shared_expert_forward_int4_nmajor)
_op(INS, "moe_forward_cutlass_nmajor_int4_full(Tensor x, Tensor logits, "
    "Tensor w13, Tensor w13_scales, Tensor w2, Tensor w2_scales, "
    "Tensor shared_gu_w, Tensor shared_d_w, Tensor shared_gate_w, "
    "int top_k, int num_shared_experts, int n_routed_experts) -> Tensor", I.moe_forward_cutlass_nmajor_int4_full)



# ---------------------------------------------------------------- GELU-tanh activation; block FP8 + 16-bit dual GEMV
def _moe_gelu_tanh_mul(input, output, N_gate_up, N_half, total_rows):
    I._chk(N_gate_up == 2 * N_half, "N_gate_up must be 2 * N_half")
    I.gelu_tanh_mul(input[:total_rows], output[:total_rows])
    return output


def _fp8_block_fp16_fused2(input, w0, s0, o0, w1, o1, block_n, block_k):
    """o0 = input @ dequant(w0, s0)^T through the block-scaled FP8 GEMV; o1 = input @ w1^T with a dense 16-bit w1
    (csrc/xpu/esimd_kernel_gemm.sycl:184-216).  The dense 16-bit half is a plain library GEMM: the reference's
    16-bit GEMV (esimd_gemv_fp16) is outside this library's quantized-linear scope."""
    _fp8_block(input, w0, s0, o0.view(input.shape[0], -1), block_n, block_k)
    I._chk(w1.dtype == input.dtype and w1.shape[1] == input.shape[1], "w1 must be a 16-bit [N1, K] matrix of the input's type")
    torch.matmul(input, w1.t(), out=o1.view(input.shape[0], -1))
    return o0


_op(NS, "esimd_moe_gelu_tanh_mul(Tensor input, Tensor output, int N_gate_up, int N_half, int total_rows) -> Tensor",
    _moe_gelu_tanh_mul)
_op(NS, "esimd_gemv_fp8_blockscale_fp16_fused2(Tensor input, Tensor w0, Tensor s0, Tensor(a!) o0, Tensor w1, Tensor(b!) o1, "
        "int block_n, int block_k) -> Tensor(a!)", _fp8_block_fp16_fused2)


# ---------------------------------------------------------------- moe_ops: FP8 (e4m3, one scale per expert) grouped MoE
MNS = "moe_ops"


def _moe_ops_topk(logits, top_k, norm):
    w, ids = I.moe_topk(logits.contiguous(), top_k, bool(norm))
    return ids, w                     # the reference returns (indices, weights) here (csrc/moe_batch/moe.sycl:1309-1345)


def _routed_fp8(x, topk_weights, topk_indices, gu_w, gu_s, dn_w, dn_s, top_k, accumulate=True):
    """Caller-supplied routing -> stable sort by expert -> grouped up (GELU-tanh * up) -> grouped down -> weighted sum
    (csrc/moe_batch/moe.sycl:2249-2340)."""
    E = gu_w.shape[0]
    ids = topk_indices.to(torch.int32).contiguous()
    offsets, tokens, _, _ = I.moe_route(ids, E)
    if accumulate:
        return I.moe_forward_full_fp8_grouped(x, gu_w, gu_s, dn_w, dn_s, topk_weights, offsets[:E], tokens, top_k, E)
    inter = I.moe_up_fp8_grouped(x, gu_w, gu_s, offsets[:E], tokens, top_k, E)
    return I.moe_down_fp8_grouped(inter, dn_w, dn_s, topk_weights, offsets[:E], tokens, top_k, E)


def _full_gelu_tanh(x, logits, gu_w, gu_s, dn_w, dn_s, top_k, n_routed_experts):
    w, ids = I.moe_topk(logits.contiguous(), top_k, True, weight_dtype=x.dtype)
    return _routed_fp8(x, w, ids, gu_w, gu_s, dn_w, dn_s, top_k)


def _full_gelu_tanh_routed(x, topk_weights, topk_indices, gu_w, gu_s, dn_w, dn_s, top_k, n_routed_experts):
    return _routed_fp8(x, topk_weights, topk_indices, gu_w, gu_s, dn_w, dn_s, top_k)


def _full_gelu_tanh_routed_no_accum(x, topk_weights, topk_indices, gu_w, gu_s, dn_w, dn_s, top_k, n_routed_experts):
    return _routed_fp8(x, topk_weights, topk_indices, gu_w, gu_s, dn_w, dn_s, top_k, accumulate=False)


def _full_gelu_tanh_decode(x, logits, gu_w, gu_s, dn_w, dn_s, per_expert_scale, top_k, n_routed_experts):
    # routing weight times the chosen expert's scale, rounded to the activation type as the reference's fold kernel
    # stores it (csrc/moe_batch/moe.sycl:2194-2201); a handful of elements, index plumbing only
    w, ids = I.moe_topk(logits.contiguous(), top_k, True, weight_dtype=x.dtype)
    w = (w.float() * per_expert_scale.float()[ids.long()]).to(x.dtype)
    return _routed_fp8(x, w, ids, gu_w, gu_s, dn_w, dn_s, top_k)


_op(MNS, "moe_accumulate(Tensor partials, int top_k, int num_shared_experts) -> Tensor", I.moe_accumulate)
_op(MNS, "moe_topk(Tensor logits, int top_k, bool norm) -> (Tensor, Tensor)", _moe_ops_topk)
_op(MNS, "moe_up_fp8_grouped(Tensor x, Tensor gate_up_weight, Tensor gate_up_scale, Tensor expert_offsets, "
         "Tensor expert_tokens, int top_k, int n_routed_experts) -> Tensor", I.moe_up_fp8_grouped)
_op(MNS, "moe_down_fp8_grouped(Tensor intermediate, Tensor down_weight, Tensor down_scale, Tensor routing_weights, "
         "Tensor expert_offsets, Tensor expert_tokens, int top_k, int n_routed_experts) -> Tensor", I.moe_down_fp8_grouped)
_op(MNS, "moe_forward_full_fp8_grouped(Tensor x, Tensor gate_up_weight, Tensor gate_up_scale, Tensor down_weight, "
         "Tensor down_scale, Tensor routing_weights, Tensor expert_offsets, Tensor expert_tokens, int top_k, "
         "int n_routed_experts) -> Tensor", I.moe_forward_full_fp8_grouped)
_op(MNS, "moe_forward_full_gelu_tanh(Tensor x, Tensor logits, Tensor gate_up_weight, Tensor gate_up_scale, "
         "Tensor down_weight, Tensor down_scale, int top_k, int n_routed_experts) -> Tensor", _full_gelu_tanh)
_op(MNS, "moe_forward_full_gelu_tanh_routed_no_accum(Tensor x, Tensor topk_weights, Tensor topk_indices, "
         "Tensor gate_up_weight, Tensor gate_up_scale, Tensor down_weight, Tensor down_scale, int top_k, "
         "int n_routed_experts) -> Tensor", _full_gelu_tanh_routed_no_accum)
_op(MNS, "moe_forward_full_gelu_tanh_routed(Tensor x, Tensor topk_weights, Tensor topk_indices, Tensor gate_up_weight, "
         "Tensor gate_up_scale, Tensor down_weight, Tensor down_scale, int top_k, int n_routed_experts) -> Tensor",
    _full_gelu_tanh_routed)
_op(MNS, "moe_forward_full_gelu_tanh_routed_decode(Tensor x, Tensor topk_weights, Tensor topk_indices, "
         "Tensor gate_up_weight, Tensor gate_up_scale, Tensor down_weight, Tensor down_scale, int top_k, "
         "int n_routed_experts) -> Tensor", _full_gelu_tanh_routed)
_op(MNS, "moe_forward_full_gelu_tanh_decode(Tensor x, Tensor logits, Tensor gate_up_weight, Tensor gate_up_scale, "
         "Tensor down_weight, Tensor down_scale, Tensor per_expert_scale, int top_k, int n_routed_experts) -> Tensor",
    _full_gelu_tanh_decode)


# ---------------------------------------------------------------- the rest of the reference's op surface
def _not_implemented(qualname):
    def fn(*args, **kwargs):
        raise RuntimeError("b2q: %s not implemented" % qualname)
    return fn


def _register_unimplemented():
    from ._surface import UNIMPLEMENTED
    for ns, schemas in UNIMPLEMENTED.items():
        lib = _lib(ns)
        for schema in schemas:
            name = schema.split("(", 1)[0]
            lib.define(schema)
            # every backend key: a call must reach the message whatever device the arguments live on
            lib.impl(name, _not_implemented("%s::%s" % (ns, name)), "CompositeExplicitAutograd")


_register_unimplemented()

REGISTERED = {ns: lib for ns, lib in _LIBS.items()}
