"""MoE pipeline oracle: routing, permutation, grouped GEMM, activation, combine."""
import torch
import torch.nn.functional as F


def topk_softmax(logits: torch.Tensor, top_k: int, renorm: bool = True, out_dtype=None):
    """fp32 softmax -> torch.topk -> renormalise -> cast (tests/test_moe_int4_kernel.py:213-216,
    python/custom_esimd_kernels_vllm/ops.py:1427-1437).  Returns (weights [T,k], ids int32 [T,k])."""
    probs = F.softmax(logits.float(), dim=-1)
    # torch.topk with the tie rule of the reference kernel made explicit: among bit-equal
    # probabilities the lowest expert index is taken first (csrc/xpu/esimd_kernels/moe_ops.h:77-104).
    # A stable descending sort does exactly that; without ties it equals torch.topk.
    sp, si = torch.sort(probs, dim=-1, descending=True, stable=True)
    w, ids = sp[..., :top_k], si[..., :top_k]
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.to(out_dtype or logits.dtype), ids.to(torch.int32)


def route(ids: torch.Tensor, num_experts: int):
    """Stable sort of the T*k (token, slot) pairs by expert (ops.py:1300-1330).

    Returns expert_offsets int32 [E+1], expert_tokens int32 [n_valid] (pair indices),
    pair_to_perm int32 [T*k] (-1 for ids outside [0, E)), rows_per_expert int32 [E].
    """
    flat = ids.reshape(-1).to(torch.int64)
    valid = (flat >= 0) & (flat < num_experts)
    key = torch.where(valid, flat, torch.full_like(flat, num_experts))
    order = torch.argsort(key, stable=True)
    n_valid = int(valid.sum())
    order = order[:n_valid]
    rows = torch.bincount(flat[valid], minlength=num_experts).to(torch.int32)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
    offsets[1:] = rows.cumsum(0)
    p2p = torch.full((flat.numel(),), -1, dtype=torch.int32)
    p2p[order] = torch.arange(n_valid, dtype=torch.int32)
    return offsets, order.to(torch.int32), p2p, rows


def silu_mul(g: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up in fp32, cast back (ops.py:1333-1342)."""
    I = g.shape[-1] // 2
    gf = g[..., :I].float()
    return ((gf / (1 + torch.exp(-gf))) * g[..., I:].float()).to(g.dtype)


def grouped_linear(x_sorted: torch.Tensor, wd: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """out[rows of e] = x[rows of e].float() @ wd[e].float().T, fp32 result (wd: [E, N, K] dequantised)."""
    out = torch.zeros(x_sorted.shape[0], wd.shape[1], dtype=torch.float32)
    for e in range(wd.shape[0]):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            out[a:b] = x_sorted[a:b].float() @ wd[e].float().T
    return out


def forward(x, logits, w13d, w2d, top_k, round_intermediates=True):
    """topk -> per expert gate_up -> SiLU*mul -> down -> weighted sum; no shared expert.

    Follows tests/test_moe_int4_kernel.py:198-247 minus the shared expert, evaluated per expert
    instead of per token.  w13d [E, 2I, H], w2d [E, H, I] are dequantised weights in x.dtype.
    With round_intermediates the gate_up result, the activation and the down result are rounded
    to x.dtype between stages, as a pipeline of separate ops with 16-bit tensors between them does.
    """
    T, H = x.shape
    E = w13d.shape[0]
    wts, ids = topk_softmax(logits, top_k, True, x.dtype)
    offsets, expert_tokens, p2p, _ = route(ids, E)
    tok = (expert_tokens // top_k).long()
    xs = x[tok]
    g = grouped_linear(xs, w13d, offsets)
    if round_intermediates:
        g = g.to(x.dtype)
    a = silu_mul(g)
    y = grouped_linear(a, w2d, offsets)
    if round_intermediates:
        y = y.to(x.dtype)
    wflat = wts.reshape(-1).float()
    yp = y.float()[p2p.long()] * wflat[:, None]
    return _ordered_sum(yp.reshape(T, top_k, H)).to(x.dtype)


def shared_expert(x, shared_gate_up, shared_down, shared_gate_w, round_intermediates=True):
    """sigmoid(x . gate_w) * down(silu(gate(x)) * up(x)) for one shared expert, fp32 result [T, H].

    tests/test_moe_int4_kernel.py:232-244.  shared_gate_up [2*Is, H] (gate rows first), shared_down [H, Is],
    shared_gate_w [1, H]; all dequantised / 16-bit weights in x.dtype.
    """
    xf = x.float()
    g = xf @ shared_gate_up.float().T
    if round_intermediates:
        g = g.to(x.dtype)
    a = silu_mul(g)
    y = a.float() @ shared_down.float().T
    if round_intermediates:
        y = y.to(x.dtype).float()
    gate = torch.sigmoid(xf @ shared_gate_w.float().T)          # [T, 1]
    return y * gate


def forward_full(x, logits, w13d, w2d, shared_gate_up, shared_down, shared_gate_w, top_k, round_intermediates=True):
    """The decode pipeline moe_forward_full_int4 computes: routed experts plus the sigmoid-gated shared expert
    (tests/test_moe_int4_kernel.py:198-247; csrc/moe_batch/moe_int4.sycl:2933-3166)."""
    routed = forward(x, logits, w13d, w2d, top_k, round_intermediates)
    sh = shared_expert(x, shared_gate_up, shared_down, shared_gate_w, round_intermediates)
    return (routed.float() + sh).to(x.dtype)


def _ordered_sum(v: torch.Tensor) -> torch.Tensor:
    acc = torch.zeros(v.shape[0], v.shape[2], dtype=torch.float32)
    for s in range(v.shape[1]):
        acc += v[:, s]
    return acc


def combine(y: torch.Tensor, wts: torch.Tensor, perm=None) -> torch.Tensor:
    """out[t] = sum_s w[t,s] * y[perm[t*k+s]] in fp32, slots in order (moe_prefill_int4.sycl:398-454)."""
    T, k = wts.shape
    idx = torch.arange(T * k) if perm is None else perm.long()
    ok = idx >= 0
    rows = y.float()[idx.clamp(min=0)] * (wts.reshape(-1).float() * ok)[:, None]
    return _ordered_sum(rows.reshape(T, k, -1)).to(y.dtype)


def gelu_tanh_mul(g: torch.Tensor) -> torch.Tensor:
    """gelu_tanh(gate) * up in fp32, cast back: 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))
    (csrc/xpu/esimd_kernels/moe_ops.h:678-723; tests/test_moe_fp8_grouped.py:5)."""
    I = g.shape[-1] // 2
    gf = g[..., :I].float()
    act = 0.5 * gf * (1.0 + torch.tanh(0.7978845608028654 * (gf + 0.044715 * gf ** 3)))
    return (act * g[..., I:].float()).to(g.dtype)


def forward_fp8_grouped(x, topk_w, topk_ids, w13q, s13, w2q, s2, accumulate=True):
    """FP8 MoE with one fp32 scale per expert and GELU-tanh, routing supplied by the caller
    (tests/test_moe_fp8_grouped.py:6-15, evaluated per expert instead of per token):
        g = x @ (decode(w13[e]) * s13[e]).T ; mid = gelu_tanh(gate) * up -> 16 bit ;
        y = (mid @ (decode(w2[e]) * s2[e]).T) * routing weight ; out[t] = sum over the token's routes.
    w13q [E, 2I, H], w2q [E, H, I] e4m3; topk_w [T, k]; topk_ids int32 [T, k].  With accumulate=False returns the
    weighted per-route rows [T * k, H] (pair order), rounded to x.dtype as the reference stores them."""
    from . import fp8
    T, H = x.shape
    k = topk_ids.shape[1]
    E = w13q.shape[0]
    offsets, expert_tokens, p2p, _ = route(topk_ids, E)
    tok = (expert_tokens // k).long()
    xs = x[tok].float()
    inter = torch.zeros(T * k, w13q.shape[1] // 2, dtype=x.dtype)
    y = torch.zeros(T * k, H, dtype=torch.float32)
    for e in range(E):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b <= a:
            continue
        g = (xs[a:b] @ (fp8.decode(w13q[e]) * float(s13[e])).T).to(x.dtype)
        mid = gelu_tanh_mul(g)
        inter[a:b] = mid
        y[a:b] = mid.float() @ (fp8.decode(w2q[e]) * float(s2[e])).T
    wflat = topk_w.reshape(-1).float()
    y_pair = y[p2p.long()]                                     # back to pair order
    if not accumulate:
        return (y_pair * wflat[:, None]).to(x.dtype)
    return _ordered_sum((y_pair.to(x.dtype).float() * wflat[:, None]).reshape(T, k, H)).to(x.dtype)
