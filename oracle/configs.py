"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark configurations.

These synthetic tensors stand in for real checkpoints: the reference's own harnesses for this path also
run on random data.  Everything is generated on the CPU from torch.manual_seed(seed).
"""
import torch
from . import int4, fp8


def _gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def int4_weight(N, K, g, scale_dtype=torch.bfloat16, lead=()):
    """Uniform nibbles in [0,15] (value-8 in [-8,7]); scales 0.002 + |N(0, 0.01)|."""
    q = torch.randint(0, 16, (*lead, N, K), generator=g, dtype=torch.uint8)
    s = (0.002 + torch.randn(*lead, N, K // 128, generator=g).abs() * 0.01).to(scale_dtype)
    return q, s


def c1(seed=0, M=16, K=4096, N=4096, dtype=torch.bfloat16):
    g = _gen(seed)
    x = torch.randn(M, K, generator=g).to(dtype)
    q, s = int4_weight(N, K, g, dtype)
    return {"x": x, "q": q, "scale": s, "w_i32": int4.pack_nmajor_i32(q)}


def c2(seed=0, M=1, N=27648, K=5120, dtype=torch.bfloat16):
    g = _gen(seed)
    w = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    wq, s = fp8.quantize_channel(w)
    x = torch.randn(M, K, generator=g).to(dtype)
    return {"x": x, "wq": wq, "scale": s}


def c3(seed=0, M=4096, N=17408, K=5120, dtype=torch.bfloat16):
    g = _gen(seed)
    w = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    wq, ws = fp8.quantize_block(w)
    x = torch.randn(M, K, generator=g).to(dtype)
    return {"x": x, "wq": wq, "ws": ws}


def c4(seed=0, T=4096, E=128, top_k=8, H=2048, I=768, dtype=torch.bfloat16):
    g = _gen(seed)
    x = torch.randn(T, H, generator=g).to(dtype)
    logits = torch.randn(T, E, generator=g).to(dtype)
    q13, s13 = int4_weight(2 * I, H, g, dtype, lead=(E,))
    q2, s2 = int4_weight(H, I, g, dtype, lead=(E,))
    return {"x": x, "logits": logits, "q13": q13, "s13": s13, "q2": q2, "s2": s2, "top_k": top_k}


C5_LAYER = {"qkv": (10240, 8192), "o": (8192, 8192), "gate_up": (57344, 8192), "down": (8192, 28672)}


def c5_layer(seed=0, M=64, tp=1, rank=0, dtype=torch.bfloat16, scale=1.0):
    """One decoder layer's four INT4 linears, sharded for tensor parallel rank `rank` of `tp`.

    Column-parallel qkv / gate_up split N (gate and up halves are each split so a rank owns
    matching slices); row-parallel o / down split K in multiples of 128.  `scale` < 1 shrinks
    every dimension for tests.
    """
    g = _gen(seed)
    out = {}
    for name, (N, K) in C5_LAYER.items():
        N, K = int(N * scale), int(K * scale)
        q, s = int4_weight(N, K, g, dtype)
        if name in ("qkv", "gate_up"):
            if name == "gate_up":
                half = N // 2
                sl = half // tp
                rows = torch.cat([torch.arange(rank * sl, (rank + 1) * sl), half + torch.arange(rank * sl, (rank + 1) * sl)])
            else:
                sl = N // tp
                rows = torch.arange(rank * sl, (rank + 1) * sl)
            q, s = q[rows], s[rows]
        else:
            sl = K // tp
            q = q[:, rank * sl:(rank + 1) * sl]
            s = s[:, rank * sl // 128:(rank + 1) * sl // 128]
        out[name] = (q.contiguous(), s.contiguous())
    out["x"] = torch.randn(M, int(8192 * scale), generator=g).to(dtype)
    return out
