"""Host side of every op: shape / dtype checks that mirror the reference's TORCH_CHECKs,
output allocation where the reference op allocates, and one call into libb2q.so.

Each function is what the matching `torch.ops.<namespace>.<op>` dispatches to for CUDA
tensors (see _register.py).  torch is used for device memory, streams and tiny index
plumbing only; all arithmetic on the path runs in libb2q.so kernels.
"""
import torch

from . import _lib as L

GROUP = 128


def _chk(cond, msg):
    if not cond:
        raise RuntimeError(msg)


# --------------------------------------------------------------------------- INT4 dense
def _int4_view(weight: torch.Tensor, scale: torch.Tensor):
    """Classify an INT4 weight/scale pair.  Returns (tensor_for_ptr, layout, N, K, s_stride_n, s_stride_g).

    Accepted presentations (all alias the formats of include/b2q.h):
      uint8 [N, K/2] / int32 [N, K/8] contiguous            -> NMAJOR
      int32 [K/8, N] with strides (1, K/8) (the .t() view)  -> NMAJOR on the same bytes
      int32 [K/8, N] contiguous with scales [K/g, N]        -> KMAJOR
    """
    _chk(weight.dim() == 2 and scale.dim() == 2, "int4 weight and scale must be 2-D")
    if weight.dtype == torch.uint8:
        _chk(weight.is_contiguous(), "uint8 int4 weight must be contiguous [N, K/2]")
        N, K = weight.shape[0], weight.shape[1] * 2
        layout, wt = L.W4_NMAJOR, weight
    elif weight.dtype == torch.int32:
        a, b = weight.shape
        if not weight.is_contiguous() and weight.stride(0) == 1 and weight.stride(1) == a:
            wt, N, K, layout = weight.t(), b, a * 8, L.W4_NMAJOR
        else:
            _chk(weight.is_contiguous(), "int4 weight must be contiguous or a transposed view of a contiguous tensor")
            nmaj = scale.shape[0] == a and scale.shape[1] * GROUP == b * 8
            kmaj = scale.shape[1] == b and scale.shape[0] * GROUP == a * 8
            if nmaj or not kmaj:
                wt, N, K, layout = weight, a, b * 8, L.W4_NMAJOR
            else:
                wt, N, K, layout = weight, b, a * 8, L.W4_KMAJOR
    else:
        raise RuntimeError("int4 weight must be uint8 or int32, got %s" % weight.dtype)
    _chk(K % GROUP == 0, "K must be a multiple of the group size 128")
    G = K // GROUP
    if tuple(scale.shape) == (N, G):
        sn, sg = scale.stride(0), scale.stride(1)
    elif tuple(scale.shape) == (G, N):
        sn, sg = scale.stride(1), scale.stride(0)
    else:
        raise RuntimeError("int4 scale shape %s does not match N=%d, K/128=%d" % (tuple(scale.shape), N, G))
    return wt, layout, N, K, sn, sg


def linear_int4(input, weight, weight_scale, output):
    L.require_cuda(input, weight, weight_scale, output)
    _chk(input.dim() == 2 and output.dim() == 2, "input/output must be 2-D")
    _chk(input.dtype in (torch.bfloat16, torch.float16), "activation must be bf16 or fp16")
    _chk(output.dtype == input.dtype, "output dtype must equal input dtype")
    wt, layout, N, K, sn, sg = _int4_view(weight, weight_scale)
    M = input.shape[0]
    _chk(input.shape[1] == K, "input K does not match weight")
    _chk(tuple(output.shape) == (M, N), "output must be [M, N]")
    _chk(input.stride(1) == 1 and output.stride(1) == 1, "input/output rows must be contiguous")
    with L.on_device(input):
        # scratch for the activation pre-pass and partial sums of the tensor-core kernels (caching allocator, no cudaMalloc)
        wsb = L.lib.b2q_linear_workspace_bytes(M, N, K)
        ws = torch.empty(wsb, dtype=torch.uint8, device=input.device)
        L.check(L.lib.b2q_linear_int4(input.data_ptr(), L.dt(input), input.stride(0) if M > 1 else K,
                                       wt.data_ptr(), layout, weight_scale.data_ptr(), L.dt(weight_scale), sn, sg,
                                       output.data_ptr(), output.stride(0) if M > 1 else N, M, N, K, GROUP,
                                       L.ptr(ws), wsb, L.stream(input)))
    return output


def linear_int4_nmajor(input, weight, weight_scale, N, K, scale_is_kmajor, output=None, signed=False):
    """out = input @ dequant(W)^T for a weight whose BYTES are the N-major [N, K/8] matrix whatever shape the tensor
    carries (the column-major repack of csrc/moe_batch/moe_int4.sycl:171-215, :3036-3040 hands over a [K/8, N]-shaped
    tensor with exactly that memory), and scales stored [K/128, N] (scale_is_kmajor) or [N, K/128].  signed: the
    nibbles are two's complement (value, not value + 8), the encoding of ops.py:1243-1263."""
    L.require_cuda(input, weight, weight_scale)
    _chk(weight.is_contiguous() and weight_scale.is_contiguous(), "weight and scale must be contiguous")
    _chk(weight.numel() * weight.element_size() * 2 == N * K, "weight bytes do not match N x K nibbles")
    G = K // GROUP
    _chk(K % GROUP == 0 and weight_scale.numel() == N * G, "scale size does not match N x K/128")
    _chk(input.dim() == 2 and input.shape[1] == K and input.stride(1) == 1, "input must be [M, K]")
    M = input.shape[0]
    if output is None:
        output = torch.empty(M, N, dtype=input.dtype, device=input.device)
    sn, sg = (1, N) if scale_is_kmajor else (G, 1)
    with L.on_device(input):
        wsb = L.lib.b2q_linear_workspace_bytes(M, N, K)
        ws = torch.empty(wsb, dtype=torch.uint8, device=input.device)
        L.check(L.lib.b2q_linear_int4(input.data_ptr(), L.dt(input), input.stride(0) if M > 1 else K,
                                       weight.data_ptr(), L.W4_NMAJOR_S4 if signed else L.W4_NMAJOR, weight_scale.data_ptr(),
                                       L.dt(weight_scale), sn, sg, output.data_ptr(), N, M, N, K, GROUP, L.ptr(ws), wsb, L.stream(input)))
    return output


def dequant_int4(weight, weight_scale, out_dtype=torch.bfloat16, layout=None):
    """Debug / bit-exactness gate: [N, K] dequantised weight."""
    L.require_cuda(weight, weight_scale)
    if layout is None:
        wt, layout, N, K, sn, sg = _int4_view(weight, weight_scale)
        _chk((layout == L.W4_NMAJOR and sg == 1) or (layout != L.W4_NMAJOR and sn == 1), "scale must be contiguous")
    else:
        wt = weight
        if layout in (L.W4_KMAJOR, L.W4_KMAJOR_MARLIN):
            N, K = weight.shape[1], weight.shape[0] * 8
        else:
            N = weight.shape[0]
            K = weight.shape[1] * (2 if weight.dtype == torch.uint8 else 8)
    out = torch.empty(N, K, dtype=out_dtype, device=weight.device)
    with L.on_device(weight):
        L.check(L.lib.b2q_dequant_int4(wt.data_ptr(), layout, weight_scale.data_ptr(), L.dt(weight_scale),
                                        out.data_ptr(), L.dt(out), N, K, GROUP, L.stream(weight)))
    return out


def resadd_rmsnorm(hidden_states, residual, norm_weight, normed_out, eps):
    """residual += hidden_states (in place); normed_out = rmsnorm(residual) * norm_weight, norm of the fp32 sum."""
    L.require_cuda(hidden_states, residual, norm_weight, normed_out)
    _chk(hidden_states.dim() == 2 and hidden_states.dtype in (torch.bfloat16, torch.float16), "hidden_states must be 2-D bf16 / fp16")
    M, K = hidden_states.shape
    for t, what in ((residual, "residual"), (normed_out, "normed_out")):
        _chk(t.dtype == hidden_states.dtype and tuple(t.shape) == (M, K) and t.is_contiguous(), what + " must be a contiguous [M, K] tensor of the activation type")
    _chk(hidden_states.is_contiguous() and norm_weight.dtype == hidden_states.dtype and norm_weight.numel() == K and norm_weight.is_contiguous(),
         "hidden_states must be contiguous and norm_weight a contiguous [K] tensor of the activation type")
    _chk(K % 8 == 0, "K must be a multiple of 8")
    with L.on_device(hidden_states):
        L.check(L.lib.b2q_resadd_rmsnorm(hidden_states.data_ptr(), residual.data_ptr(), norm_weight.data_ptr(), normed_out.data_ptr(),
                                          L.dt(hidden_states), M, K, float(eps), L.stream(hidden_states)))


def rmsnorm_fused(hidden_states, residual, scalar, w1, out1, w2, out2, eps):
    """v = (hidden + residual) * scalar (residual <- v) or v = residual when hidden_states is None;
    out1 = rmsnorm(v) * w1 and, when w2 / out2 are given, out2 = rmsnorm(v) * w2 (b2q_rmsnorm_fused)."""
    L.require_cuda(residual, w1, out1)
    _chk(residual.dim() == 2 and residual.dtype in (torch.bfloat16, torch.float16) and residual.is_contiguous(),
         "residual must be a contiguous 2-D bf16 / fp16 tensor")
    M, K = residual.shape
    _chk(K % 8 == 0, "K must be a multiple of 8")
    for t, what in ((hidden_states, "hidden_states"), (out1, "out1"), (out2, "out2")):
        if t is not None:
            _chk(t.dtype == residual.dtype and tuple(t.shape) == (M, K) and t.is_contiguous(),
                 what + " must be a contiguous [M, K] tensor of the activation type")
    for t, what in ((w1, "w1"), (w2, "w2")):
        if t is not None:
            _chk(t.dtype == residual.dtype and t.numel() == K and t.is_contiguous(), what + " must be a contiguous [K] tensor")
    _chk((w2 is None) == (out2 is None), "w2 and out2 go together")
    with L.on_device(residual):
        L.check(L.lib.b2q_rmsnorm_fused(L.ptr(hidden_states), residual.data_ptr(), float(scalar), w1.data_ptr(),
                                         out1.data_ptr(), L.ptr(w2), L.ptr(out2), L.dt(residual), M, K, float(eps),
                                         L.stream(residual)))


def gated_rmsnorm(x, z, norm_weight, eps):
    """rmsnorm(x) * norm_weight * silu(z) per row of x [rows, V]; returns a new [1, rows * V] tensor."""
    L.require_cuda(x, z, norm_weight)
    _chk(x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16), "x must be 2-D bf16 / fp16")
    rows, V = x.shape
    _chk(z.dtype == x.dtype and tuple(z.shape) == (rows, V) and x.is_contiguous() and z.is_contiguous(), "x and z must be contiguous [rows, V]")
    _chk(norm_weight.dtype == x.dtype and norm_weight.numel() == V and norm_weight.is_contiguous(), "norm_weight must be a contiguous [V] tensor")
    out = torch.empty(1, rows * V, dtype=x.dtype, device=x.device)
    with L.on_device(x):
        L.check(L.lib.b2q_gated_rmsnorm(x.data_ptr(), z.data_ptr(), norm_weight.data_ptr(), out.data_ptr(), L.dt(x), rows, V,
                                         float(eps), L.stream(x)))
    return out


def q4_0_quantize(input, out_qweight, out_scale):
    """GGML Q4_0, group 128: fills out_qweight int32 [M, K/8] and out_scale fp16 [M, K/128] in place."""
    L.require_cuda(input, out_qweight, out_scale)
    _chk(input.dim() == 2 and input.dtype in (torch.bfloat16, torch.float16), "input must be a 2-D bf16 / fp16 tensor")
    M, K = input.shape
    _chk(K % 128 == 0 and input.stride(1) == 1, "K must be a multiple of 128 and rows contiguous")
    _chk(out_qweight.dtype == torch.int32 and tuple(out_qweight.shape) == (M, K // 8) and out_qweight.is_contiguous(),
         "out_qweight must be a contiguous int32 [M, K/8] tensor")
    _chk(out_scale.dtype == torch.float16 and tuple(out_scale.shape) == (M, K // 128) and out_scale.is_contiguous(),
         "out_scale must be a contiguous fp16 [M, K/128] tensor")
    with L.on_device(input):
        L.check(L.lib.b2q_quantize_q4_0(input.data_ptr(), L.dt(input), input.stride(0) if M > 1 else K,
                                         out_qweight.data_ptr(), out_scale.data_ptr(), M, K, L.stream(input)))


# --------------------------------------------------------------------------- FP8 dense
def linear_fp8(input, weight, weight_scale, output, scale_mode, N=None, K=None):
    L.require_cuda(input, weight, weight_scale, output)
    _chk(input.dim() == 2 and output.dim() == 2 and weight.dim() == 2, "input/weight/output must be 2-D")
    _chk(input.dtype in (torch.bfloat16, torch.float16), "activation must be bf16 or fp16")
    _chk(output.dtype == input.dtype, "output dtype must equal input dtype")
    _chk(weight.is_contiguous(), "fp8 weight must be a contiguous [N, K] tensor (a transposed view is read wrongly)")
    wn, wk = weight.shape
    _chk((N is None or N == wn) and (K is None or K == wk), "N/K do not match the weight shape")
    M = input.shape[0]
    _chk(input.shape[1] == wk and tuple(output.shape) == (M, wn), "shape mismatch")
    _chk(input.stride(1) == 1 and output.stride(1) == 1, "input/output rows must be contiguous")
    if scale_mode == L.SCALE_CHANNEL:
        _chk(weight_scale.numel() == wn and weight_scale.is_contiguous(), "per-channel scale must have N elements")
    elif scale_mode == L.SCALE_TENSOR:
        _chk(weight_scale.numel() == 1 and weight_scale.dtype == torch.float32, "per-tensor scale must be one fp32")
    else:
        _chk(weight_scale.dtype == torch.float32 and weight_scale.is_contiguous(), "block scale must be fp32")
        _chk(tuple(weight_scale.shape) == ((wn + 127) // 128, (wk + 127) // 128), "block scale shape mismatch")
    with L.on_device(input):
        ws, wsb = None, 0
        if input.dtype == torch.bfloat16 or M <= 64:
            # scratch for the activation pre-pass and partial sums (torch's caching allocator: no cudaMalloc in steady state)
            wsb = L.lib.b2q_linear_fp8_workspace_bytes(M, wn, wk)
            ws = torch.empty(wsb, dtype=torch.uint8, device=input.device)
        L.check(L.lib.b2q_linear_fp8(input.data_ptr(), L.dt(input), input.stride(0) if M > 1 else wk,
                                      weight.data_ptr(), L.fp8_fmt(weight), weight_scale.data_ptr(),
                                      L.dt(weight_scale), scale_mode, output.data_ptr(),
                                      output.stride(0) if M > 1 else wn, M, wn, wk, L.ptr(ws), wsb, L.stream(input)))
    return output


def resadd_norm_linear_fp8(hidden_states, residual, norm_weight, normed_out, eps, scalar, weight, weight_scale, output,
                           scale_mode):
    """residual <- (hidden + residual) * scalar; normed_out <- rmsnorm(residual) * norm_weight; output <- normed_out @ W^T
    (b2q_resadd_norm_linear_fp8: on the decode path the norm runs inside the GEMV's activation pre-pass)."""
    L.require_cuda(hidden_states, residual, norm_weight, normed_out, weight, weight_scale, output)
    _chk(hidden_states.dim() == 2 and hidden_states.dtype in (torch.bfloat16, torch.float16), "hidden_states must be 2-D bf16 / fp16")
    M, K = hidden_states.shape
    for t, what in ((hidden_states, "hidden_states"), (residual, "residual"), (normed_out, "normed_out")):
        _chk(t.dtype == hidden_states.dtype and tuple(t.shape) == (M, K) and t.is_contiguous(), what + " must be a contiguous [M, K] tensor of the activation type")
    _chk(norm_weight.dtype == hidden_states.dtype and norm_weight.numel() == K and norm_weight.is_contiguous(), "norm_weight must be a contiguous [K] tensor")
    _chk(weight.dim() == 2 and weight.is_contiguous() and weight.shape[1] == K, "fp8 weight must be a contiguous [N, K] tensor")
    N = weight.shape[0]
    _chk(tuple(output.shape) == (M, N) and output.dtype == hidden_states.dtype and output.stride(1) == 1, "output must be [M, N] of the activation type")
    with L.on_device(hidden_states):
        wsb = L.lib.b2q_linear_fp8_workspace_bytes(M, N, K)
        ws = torch.empty(wsb, dtype=torch.uint8, device=hidden_states.device)
        L.check(L.lib.b2q_resadd_norm_linear_fp8(hidden_states.data_ptr(), residual.data_ptr(), norm_weight.data_ptr(),
                                                  normed_out.data_ptr(), float(eps), float(scalar), L.dt(hidden_states),
                                                  weight.data_ptr(), L.fp8_fmt(weight), weight_scale.data_ptr(), L.dt(weight_scale),
                                                  scale_mode, output.data_ptr(), output.stride(0) if M > 1 else N, M, N, K,
                                                  L.ptr(ws), wsb, L.stream(hidden_states)))
    return output


def dequant_fp8(weight, weight_scale, scale_mode, out_dtype=torch.float32):
    L.require_cuda(weight, weight_scale)
    N, K = weight.shape
    out = torch.empty(N, K, dtype=out_dtype, device=weight.device)
    with L.on_device(weight):
        L.check(L.lib.b2q_dequant_fp8(weight.data_ptr(), L.fp8_fmt(weight), weight_scale.data_ptr(),
                                       L.dt(weight_scale), scale_mode, out.data_ptr(), L.dt(out), N, K,
                                       L.stream(weight)))
    return out


def quantize_fp8(w, scale_mode):
    """e4m3 weight quantisation on the device: (wq [N, K] float8_e4m3fn, scale fp32) with the scale shape of scale_mode:
    [N] per channel, [1] per tensor, [ceil(N/128), ceil(K/128)] per block (b2q_quantize_fp8)."""
    L.require_cuda(w)
    _chk(w.dim() == 2 and w.stride(1) == 1 and w.dtype in (torch.bfloat16, torch.float16, torch.float32),
         "weight must be a 2-D bf16 / fp16 / fp32 tensor with contiguous rows")
    N, K = w.shape
    shape = {L.SCALE_CHANNEL: (N,), L.SCALE_TENSOR: (1,), L.SCALE_BLOCK128: ((N + 127) // 128, (K + 127) // 128)}[scale_mode]
    wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device=w.device)
    scale = torch.empty(shape, dtype=torch.float32, device=w.device)
    dt = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[w.dtype]
    with L.on_device(w):
        L.check(L.lib.b2q_quantize_fp8(w.data_ptr(), dt, w.stride(0), wq.data_ptr(), scale.data_ptr(), scale_mode, N, K,
                                        L.stream(w)))
    return wq, scale


def act_quant_fp8_1x128(x):
    L.require_cuda(x)
    M, K = x.shape
    _chk(K % 128 == 0 and x.stride(1) == 1, "K must be a multiple of 128 and rows contiguous")
    xq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    xs = torch.empty(M, K // 128, dtype=torch.float32, device=x.device)
    with L.on_device(x):
        L.check(L.lib.b2q_act_quant_fp8_1x128(x.data_ptr(), L.dt(x), x.stride(0) if M > 1 else K, xq.data_ptr(),
                                               xs.data_ptr(), M, K, L.stream(x)))
    return xq, xs


def gemm_fp8_block_w8a8(xq, xs, weight, weight_scale, output):
    L.require_cuda(xq, xs, weight, weight_scale, output)
    M, K = xq.shape
    N = weight.shape[0]
    _chk(weight.shape[1] == K and tuple(output.shape) == (M, N), "shape mismatch")
    _chk(xq.is_contiguous() and xs.is_contiguous() and weight.is_contiguous() and weight_scale.is_contiguous(),
         "operands must be contiguous")
    with L.on_device(xq):
        L.check(L.lib.b2q_gemm_fp8_block_w8a8(xq.data_ptr(), xs.data_ptr(), weight.data_ptr(),
                                               weight_scale.data_ptr(), output.data_ptr(), L.dt(output),
                                               output.stride(0), M, N, K, L.stream(xq)))
    return output


# --------------------------------------------------------------------------- MoE pieces
def moe_topk(logits, top_k, renorm=True, weights=None, ids=None, weight_dtype=None):
    L.require_cuda(logits)
    _chk(logits.dim() == 2 and logits.is_contiguous(), "router logits must be contiguous [T, E]")
    T, E = logits.shape
    if weights is None:
        weights = torch.empty(T, top_k, dtype=weight_dtype or logits.dtype, device=logits.device)
    if ids is None:
        ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    _chk(ids.dtype == torch.int32 and ids.is_contiguous() and weights.is_contiguous(), "bad top-k outputs")
    with L.on_device(logits):
        L.check(L.lib.b2q_moe_topk(logits.data_ptr(), L.dt(logits), T, E, top_k, 1 if renorm else 0,
                                    weights.data_ptr(), L.dt(weights), ids.data_ptr(), L.stream(logits)))
    return weights, ids


def moe_route(ids, num_experts):
    """Returns expert_offsets [E+1], expert_tokens [T*k], pair_to_perm [T*k], rows_per_expert [E] (all int32)."""
    L.require_cuda(ids)
    _chk(ids.dtype == torch.int32 and ids.is_contiguous(), "expert ids must be contiguous int32")
    n = ids.numel()
    dev = ids.device
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    tokens = torch.empty(n, dtype=torch.int32, device=dev)
    p2p = torch.empty(n, dtype=torch.int32, device=dev)
    rows = torch.empty(num_experts, dtype=torch.int32, device=dev)
    wsb = L.lib.b2q_moe_route_workspace_bytes(n, num_experts)
    ws = torch.empty(wsb, dtype=torch.uint8, device=dev)
    with L.on_device(ids):
        L.check(L.lib.b2q_moe_route(ids.data_ptr(), n, num_experts, offsets.data_ptr(), tokens.data_ptr(),
                                     p2p.data_ptr(), rows.data_ptr(), ws.data_ptr(), wsb, L.stream(ids)))
    return offsets, tokens, p2p, rows


def gather_rows(src, idx, div, rows=None):
    L.require_cuda(src)
    _chk(src.dim() == 2 and src.is_contiguous(), "source must be contiguous 2-D")
    rows = idx.numel() if rows is None else rows
    out = torch.empty(rows, src.shape[1], dtype=src.dtype, device=src.device)
    with L.on_device(src):
        L.check(L.lib.b2q_gather_rows(src.data_ptr(), L.ptr(idx), div, out.data_ptr(), rows, src.shape[1],
                                       src.element_size(), L.stream(src)))
    return out


def silu_mul(gate_up, out=None):
    L.require_cuda(gate_up)
    _chk(gate_up.dim() == 2 and gate_up.is_contiguous(), "gate_up must be contiguous [rows, 2I]")
    rows, two_i = gate_up.shape
    if out is None:
        out = torch.empty(rows, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    with L.on_device(gate_up):
        L.check(L.lib.b2q_silu_mul(gate_up.data_ptr(), out.data_ptr(), L.dt(gate_up), rows, two_i // 2,
                                    L.stream(gate_up)))
    return out


def gelu_tanh_mul(gate_up, out=None):
    L.require_cuda(gate_up)
    _chk(gate_up.dim() == 2 and gate_up.is_contiguous(), "gate_up must be contiguous [rows, 2I]")
    rows, two_i = gate_up.shape
    if out is None:
        out = torch.empty(rows, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    with L.on_device(gate_up):
        L.check(L.lib.b2q_gelu_tanh_mul(gate_up.data_ptr(), out.data_ptr(), L.dt(gate_up), rows, two_i // 2,
                                         L.stream(gate_up)))
    return out


def moe_combine(y, weights, perm, T, top_k, out=None, w_by_row=False):
    """out[t] = sum_s weights[t, s] * y[row(t, s)] in fp32; weights=None adds the rows unweighted."""
    L.require_cuda(y, weights)
    _chk(y.dim() == 2 and y.is_contiguous() and (weights is None or weights.is_contiguous()), "combine operands must be contiguous")
    H = y.shape[1]
    if out is None:
        out = torch.empty(T, H, dtype=y.dtype, device=y.device)
    with L.on_device(y):
        L.check(L.lib.b2q_moe_combine(y.data_ptr(), L.ptr(weights), L.dt(weights) if weights is not None else 0, L.ptr(perm),
                                       out.data_ptr(), L.dt(y), T, top_k, H, 1 if w_by_row else 0, L.stream(y)))
    return out


def _moe_int4_layout(weight, scale, K):
    """Stacked expert weights: int32 [E, N, K/8] / uint8 [E, N, K/2] (N-major) or int32 [E, K/8, N] (K-major)."""
    _chk(weight.dim() == 3 and scale.dim() == 3 and weight.is_contiguous() and scale.is_contiguous(),
         "expert weights and scales must be contiguous 3-D")
    if weight.dtype == torch.uint8:
        _chk(weight.shape[2] * 2 == K, "uint8 expert weight must be [E, N, K/2]")
        return weight.shape[1], None
    _chk(weight.dtype == torch.int32, "expert weight must be int32 or uint8")
    if weight.shape[2] * 8 == K and scale.shape[1] == weight.shape[1] and scale.shape[2] * GROUP == K:
        return weight.shape[1], False
    _chk(weight.shape[1] * 8 == K and scale.shape[2] == weight.shape[2] and scale.shape[1] * GROUP == K,
         "expert weight / scale shapes do not match K=%d" % K)
    return weight.shape[2], True


def moe_gemm_int4(x, weight, scale, expert_offsets, rows, *, row_map=None, row_div=1, out_map=None, act=L.ACT_NONE,
                  out_rows=None, layout=None):
    """Grouped INT4 GEMM over expert-sorted rows (see b2q_moe_gemm_int4 in include/b2q.h).

    act=ACT_SILU_MUL_IN: x is the un-activated [rows, 2K] gate_up result and the GEMM runs on silu(gate) * up.
    """
    L.require_cuda(x, weight, scale, expert_offsets)
    _chk(x.dim() == 2 and x.stride(1) == 1, "x rows must be contiguous")
    K = x.shape[1] // 2 if act == L.ACT_SILU_MUL_IN else x.shape[1]
    N, kmajor = _moe_int4_layout(weight, scale, K)
    if layout is None:
        layout = L.W4_NMAJOR if not kmajor else L.W4_KMAJOR_MARLIN
    E = weight.shape[0]
    _chk(expert_offsets.dtype == torch.int32 and expert_offsets.numel() == E + 1, "expert_offsets must be int32 [E+1]")
    n_out = N // 2 if act == L.ACT_SILU_MUL else N
    out = torch.empty(out_rows if out_rows is not None else rows, n_out, dtype=x.dtype, device=x.device)
    wsb = L.lib.b2q_moe_gemm_workspace_bytes(rows, E, N, K, act, 1 if row_map is not None else 0)
    ws = torch.empty(wsb, dtype=torch.uint8, device=x.device)
    with L.on_device(x):
        L.check(L.lib.b2q_moe_gemm_int4(x.data_ptr(), L.dt(x), x.stride(0), L.ptr(row_map), row_div,
                                         weight.data_ptr(), layout, scale.data_ptr(), L.dt(scale),
                                         expert_offsets.data_ptr(), E, out.data_ptr(), n_out, L.ptr(out_map),
                                         rows, N, K, GROUP, act, ws.data_ptr(), wsb, L.stream(x)))
    return out


def moe_gemm_fp8(x, weight, scale, expert_offsets, rows, scale_mode, *, out=None, row_map=None, row_div=1,
                 out_map=None, act=L.ACT_NONE):
    L.require_cuda(x, weight, scale, expert_offsets)
    _chk(x.dim() == 2 and x.stride(1) == 1 and weight.dim() == 3 and weight.is_contiguous(), "bad operands")
    E, N, K = weight.shape
    _chk(x.shape[1] == K, "K mismatch")
    _chk(scale.dtype == torch.float32 and scale.is_contiguous(), "scales must be contiguous fp32")
    if expert_offsets.dtype != torch.int32:
        expert_offsets = expert_offsets.view(torch.int32) if expert_offsets.element_size() == 4 else expert_offsets.to(torch.int32)
    _chk(expert_offsets.numel() == E + 1, "expert_idx must have E+1 entries")
    n_out = N // 2 if act in (L.ACT_SILU_MUL, L.ACT_GELU_TANH_MUL) else N
    if out is None:
        out = torch.empty(rows, n_out, dtype=x.dtype, device=x.device)
    wsb = L.lib.b2q_moe_gemm_workspace_bytes(rows, E, N, K, act, 1 if row_map is not None else 0)
    ws = torch.empty(wsb, dtype=torch.uint8, device=x.device)
    with L.on_device(x):
        L.check(L.lib.b2q_moe_gemm_fp8(x.data_ptr(), L.dt(x), x.stride(0), L.ptr(row_map), row_div,
                                        weight.data_ptr(), L.fp8_fmt(weight), scale.data_ptr(), scale_mode,
                                        expert_offsets.data_ptr(), E, out.data_ptr(), out.stride(0), L.ptr(out_map),
                                        rows, N, K, act, ws.data_ptr(), wsb, L.stream(x)))
    return out


def moe_forward_int4(x, logits, w13, s13, w2, s2, top_k, num_experts, layout=None):
    """topk -> route -> gate_up GEMM + SiLU*mul -> down GEMM -> weighted combine (no shared expert).

    The pipeline of moe_prefill_full_int4 (csrc/moe_prefill/moe_prefill_int4.sycl:920-988).  The
    activations are never materialised in expert order: the up GEMM gathers token rows through
    expert_tokens and the combine reads the down result through pair_to_perm.
    """
    T = x.shape[0]
    wts, ids = moe_topk(logits, top_k, True, weight_dtype=x.dtype)
    offsets, tokens, p2p, _ = moe_route(ids, num_experts)
    rows = T * top_k
    gate_up = moe_gemm_int4(x, w13, s13, offsets, rows, row_map=tokens, row_div=top_k, layout=layout)
    y = moe_gemm_int4(gate_up, w2, s2, offsets, rows, act=L.ACT_SILU_MUL_IN, layout=layout)
    return moe_combine(y, wts, p2p, T, top_k)


def moe_shared_gate_add(x, gate_w, shared, routed, out=None):
    """out = routed + sigmoid(x . gate_w) * shared (b2q_moe_shared_gate_add)."""
    L.require_cuda(x, gate_w, shared, routed)
    T, H = x.shape
    _chk(x.is_contiguous() and shared.is_contiguous() and routed.is_contiguous(), "operands must be contiguous")
    _chk(gate_w.numel() == H and gate_w.is_contiguous() and gate_w.dtype == x.dtype, "gate weight must be [1, H] in x's dtype")
    _chk(tuple(shared.shape) == (T, H) and tuple(routed.shape) == (T, H), "shared / routed must be [T, H]")
    if out is None:
        out = torch.empty_like(routed)
    with L.on_device(x):
        L.check(L.lib.b2q_moe_shared_gate_add(x.data_ptr(), gate_w.data_ptr(), shared.data_ptr(), routed.data_ptr(),
                                               out.data_ptr(), L.dt(x), T, H, L.stream(x)))
    return out


def moe_router_forward_int4(x, weight, scale, use_ggml_layout):
    """Router logits x @ dequant(Wg)^T, [T, E] (moe_router_forward_int4, csrc/moe_batch/moe_int4.sycl:171-260).

    GGML layout: weight uint8 [E, K/2] or int32 [E, K/8], scale [E, K/128].  Otherwise the weight may arrive shaped
    [K/8, E] after the column-major repack (its memory is still [E, K/8]) with scale [K/128, E].
    """
    _chk(x.dim() == 2 and x.is_contiguous(), "x must be contiguous [T, K]")
    K = x.shape[1]
    E = weight.numel() * weight.element_size() * 2 // K
    G = K // GROUP
    if use_ggml_layout:
        _chk(tuple(scale.shape) == (E, G), "gate scale must be [E, K/128]")
        return linear_int4_nmajor(x, weight, scale, E, K, False)
    kmaj = tuple(scale.shape) == (G, E) or scale.numel() == G * E
    _chk(kmaj, "gate scale must hold K/128 x E values")
    return linear_int4_nmajor(x, weight, scale.contiguous(), E, K, True)


def moe_shared_expert_int4(x, gu_w, gu_s, down_w, down_s, gate_w, scale_is_kmajor, signed=False):
    """sigmoid(x . gate_w) * down(silu(gate(x)) * up(x)) with N-major INT4 weights, returned un-added: [T, H] shared
    output and the gate is applied by moe_shared_gate_add."""
    K = x.shape[1]
    two_i = gu_w.numel() * gu_w.element_size() * 2 // K
    g = linear_int4_nmajor(x, gu_w, gu_s, two_i, K, scale_is_kmajor, signed=signed)
    a = silu_mul(g)
    return linear_int4_nmajor(a, down_w, down_s, K, two_i // 2, scale_is_kmajor, signed=signed)


def moe_shared_expert_forward_int4_nmajor(x, gate_up_qweight, gate_up_scale, down_qweight, down_scale, gate_weight):
    """moe_shared_expert_forward_int4_nmajor (csrc/moe_batch/moe_int4.sycl:3311-3366; ops.py:1209-1230): uint8
    [2I, H/2] / [H, I/2] two's-complement nibbles with [N, K/128] scales; returns the sigmoid-gated shared expert
    output [T, H]."""
    _chk(gate_weight.shape[0] == 1, "one shared expert is supported")
    _chk(gate_up_qweight.dtype == torch.uint8 and down_qweight.dtype == torch.uint8, "weights must be uint8 nibble pairs")
    x = x.contiguous()
    y = moe_shared_expert_int4(x, gate_up_qweight, gate_up_scale, down_qweight, down_scale, gate_weight, False,
                               signed=True)
    return moe_shared_gate_add(x, gate_weight.contiguous(), y, torch.zeros_like(y))


def moe_forward_full_int4(x, logits, gate_up_qweight, gate_up_scales, shared_gate_up_weight, shared_gate_up_scale,
                          down_qweight, down_scales, shared_down_weight, shared_down_scale, shared_expert_gate_weight,
                          top_k, num_shared_experts, n_routed_experts, use_ggml_layout=False):
    """Decode pipeline with the sigmoid-gated shared expert (moe_forward_full_int4,
    csrc/moe_batch/moe_int4.sycl:2933-3166; python ops.py:1171-1206).

    Routed experts: K-major marlin-shuffled int32 [E, K/8, N] with scales [E, K/128, N], or, with use_ggml_layout,
    N-major [E, N, K/8] with scales [E, N, K/128].  Shared expert: INT4 (int32, column-major repacked, scales
    [K/128, N]) or 16-bit dense [2*Is, H] / [H, Is], told apart by dtype as the reference does (:2965).  The dense
    16-bit shared expert is a plain library GEMM (torch.nn.functional.linear); everything else runs in this library.
    """
    _chk(num_shared_experts in (0, 1), "0 or 1 shared experts are supported")
    x = x.contiguous()
    layout = L.W4_NMAJOR if use_ggml_layout else L.W4_KMAJOR_MARLIN
    routed = moe_forward_int4(x, logits.contiguous(), gate_up_qweight, gate_up_scales, down_qweight, down_scales,
                              top_k, n_routed_experts, layout=layout)
    if num_shared_experts == 0 or shared_gate_up_weight.numel() == 0:
        return routed
    if shared_gate_up_weight.dtype in (torch.int32, torch.uint8):
        y = moe_shared_expert_int4(x, shared_gate_up_weight, shared_gate_up_scale, shared_down_weight,
                                   shared_down_scale, shared_expert_gate_weight, True)
    else:
        g = torch.nn.functional.linear(x, shared_gate_up_weight.to(x.dtype))
        y = torch.nn.functional.linear(silu_mul(g), shared_down_weight.to(x.dtype)).contiguous()
    return moe_shared_gate_add(x, shared_expert_gate_weight.to(x.dtype).contiguous(), y, routed, out=routed)


def moe_forward_cutlass_nmajor_int4_full(x, logits, w13, w13_scales, w2, w2_scales, shared_gu_w, shared_d_w,
                                         shared_gate_w, top_k, num_shared_experts, n_routed_experts):
    """moe_forward_cutlass_nmajor_int4_full (csrc/moe_batch/moe_int4.sycl:3702-3770): routed experts as two's-complement
    N-major nibbles uint8 [E, N, K/2] (ops.py:1243-1297) with scales [E, N, K/128], 16-bit dense shared expert."""
    _chk(num_shared_experts in (0, 1), "0 or 1 shared experts are supported")
    x = x.contiguous()
    routed = moe_forward_int4(x, logits.contiguous(), w13, w13_scales, w2, w2_scales, top_k, n_routed_experts,
                              layout=L.W4_NMAJOR_S4)
    if num_shared_experts == 0 or shared_gu_w.numel() == 0:
        return routed
    sg = shared_gu_w[0] if shared_gu_w.dim() == 3 else shared_gu_w
    sd = shared_d_w[0] if shared_d_w.dim() == 3 else shared_d_w
    sw = shared_gate_w[0] if shared_gate_w.dim() == 3 else shared_gate_w
    g = torch.nn.functional.linear(x, sg.to(x.dtype))
    y = torch.nn.functional.linear(silu_mul(g), sd.to(x.dtype)).contiguous()
    return moe_shared_gate_add(x, sw.to(x.dtype).contiguous(), y, routed, out=routed)


# --------------------------------------------------------------------------- FP8 grouped MoE (moe_ops namespace)
def _offsets_closed(expert_offsets, total):
    """The reference's gather returns E exclusive-prefix entries; the grouped GEMM wants the closing E+1-th too."""
    tail = torch.full((1,), total, dtype=torch.int32, device=expert_offsets.device)
    return torch.cat([expert_offsets.to(torch.int32), tail])


def _fp8_experts(w):
    _chk(w.dim() == 3 and w.is_contiguous(), "expert weights must be contiguous [E, N, K]")
    return w.view(torch.float8_e4m3fn) if w.dtype in (torch.uint8, torch.int8) else w


def moe_up_fp8_grouped(x, gate_up_weight, gate_up_scale, expert_offsets, expert_tokens, top_k, n_routed_experts):
    """moe_ops.moe_up_fp8_grouped (csrc/moe_batch/moe_fp8_grouped.h:247-291): e4m3 [E, 2I, H] weights with one fp32
    scale per expert, token rows gathered through expert_tokens (pair = token * top_k + slot), GELU-tanh(gate) * up,
    result rows indexed by pair: [T * top_k, I]."""
    L.require_cuda(x, gate_up_weight, gate_up_scale, expert_offsets, expert_tokens)
    w = _fp8_experts(gate_up_weight)
    _chk(w.shape[0] == n_routed_experts and gate_up_scale.numel() == n_routed_experts, "one scale per expert")
    total = x.shape[0] * top_k
    _chk(expert_tokens.numel() == total and expert_tokens.dtype == torch.int32, "expert_tokens must be int32 [T * top_k]")
    off = _offsets_closed(expert_offsets, total)
    return moe_gemm_fp8(x.contiguous(), w, gate_up_scale.float().contiguous(), off, total, L.SCALE_TENSOR,
                        row_map=expert_tokens, row_div=top_k, out_map=expert_tokens, act=L.ACT_GELU_TANH_MUL)


def moe_down_fp8_grouped(intermediate, down_weight, down_scale, routing_weights, expert_offsets, expert_tokens, top_k,
                         n_routed_experts, weighted=True):
    """moe_ops.moe_down_fp8_grouped (csrc/moe_batch/moe_fp8_grouped.h:293-335): per-route output rows [T * top_k, H],
    indexed by pair and multiplied by the pair's routing weight."""
    L.require_cuda(intermediate, down_weight, down_scale, expert_offsets, expert_tokens)
    w = _fp8_experts(down_weight)
    total = intermediate.shape[0]
    off = _offsets_closed(expert_offsets, total)
    y = moe_gemm_fp8(intermediate.contiguous(), w, down_scale.float().contiguous(), off, total, L.SCALE_TENSOR,
                     row_map=expert_tokens, row_div=1, out_map=expert_tokens)
    if weighted:
        rw = routing_weights.reshape(-1).contiguous()
        _chk(rw.numel() == total, "routing_weights must hold one weight per (token, slot) pair")
        moe_combine(y, rw, None, total, 1, out=y)            # row t scaled by rw[t], in place
    return y


def moe_forward_full_fp8_grouped(x, gate_up_weight, gate_up_scale, down_weight, down_scale, routing_weights,
                                 expert_offsets, expert_tokens, top_k, n_routed_experts):
    """moe_ops.moe_forward_full_fp8_grouped (csrc/moe_batch/moe_fp8_grouped.h:370-400): up, down and the sum over a
    token's top_k routes in one call.  The routing weight is applied inside the fp32 sum (one rounding) instead of
    to the 16-bit per-route rows."""
    T = x.shape[0]
    inter = moe_up_fp8_grouped(x, gate_up_weight, gate_up_scale, expert_offsets, expert_tokens, top_k, n_routed_experts)
    y = moe_down_fp8_grouped(inter, down_weight, down_scale, None, expert_offsets, expert_tokens, top_k,
                             n_routed_experts, weighted=False)
    rw = routing_weights.reshape(-1).contiguous()
    _chk(rw.numel() == T * top_k, "routing_weights must hold one weight per (token, slot) pair")
    return moe_combine(y, rw, None, T, top_k)


def moe_accumulate(partials, top_k, num_shared_experts):
    """moe_ops.moe_accumulate (csrc/moe_batch/moe.sycl:1177-1230): out[t] = sum of the token's top_k + num_shared
    consecutive rows of partials, fp32 sum, one rounding."""
    L.require_cuda(partials)
    rpt = top_k + num_shared_experts
    _chk(partials.dim() == 2 and partials.is_contiguous() and partials.shape[0] % rpt == 0, "partials must be [T * rows_per_token, H]")
    return moe_combine(partials, None, None, partials.shape[0] // rpt, rpt)
