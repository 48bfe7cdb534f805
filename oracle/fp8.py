"""FP8 formats: exact decode tables, quantisers (per-channel / per-tensor / 128x128 / 1x128), linear oracles."""
import numpy as np
import torch

FP8_MAX = 448.0
BLOCK = 128


def e4m3_table() -> np.ndarray:
    """All 256 e4m3fn codes decoded from the format definition (bias 7, no inf, 0x7f/0xff NaN)."""
    out = np.empty(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 7
        if e == 0:
            v = m * 2.0 ** -9
        elif e == 15 and m == 7:
            v = np.nan
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        out[b] = s * v
    return out


def e5m2_table() -> np.ndarray:
    """All 256 e5m2 codes: the high byte of an IEEE fp16."""
    return (np.arange(256, dtype=np.uint16) << 8).view(np.float16).astype(np.float32)


def decode(w: torch.Tensor, e5m2: bool = False) -> torch.Tensor:
    """uint8 / float8 tensor -> fp32 via the table (exact, subnormals kept)."""
    tab = torch.from_numpy(e5m2_table() if e5m2 else e4m3_table())
    return tab[w.view(torch.uint8).to(torch.int64)]


def quantize_channel(w: torch.Tensor):
    """Per-output-row scale = amax / 448 (fp32, clamp 1e-12); Wq = (W / s).to(e4m3)."""
    wf = w.float()
    s = (wf.abs().amax(dim=1).clamp(min=1e-12) / FP8_MAX).to(torch.float32)
    return (wf / s[:, None]).to(torch.float8_e4m3fn), s


def quantize_tensor(w: torch.Tensor):
    wf = w.float()
    s = (wf.abs().max().clamp(min=1e-12) / FP8_MAX).to(torch.float32).reshape(1)
    return (wf / s).to(torch.float8_e4m3fn), s


def quantize_block(w: torch.Tensor, bn: int = BLOCK, bk: int = BLOCK):
    """128x128 block quantiser, tests/test_fp8_blockscale_gemm.py:13-28 (vectorised; same arithmetic).

    Accepts [..., N, K]; partial edge blocks own their remainder.
    """
    wf = w.float()
    lead = wf.shape[:-2]
    N, K = wf.shape[-2:]
    Nb, Kb = (N + bn - 1) // bn, (K + bk - 1) // bk
    pad = torch.zeros(*lead, Nb * bn, Kb * bk)
    pad[..., :N, :K] = wf
    blk = pad.reshape(*lead, Nb, bn, Kb, bk)
    amax = blk.abs().amax(dim=(-3, -1)).clamp(min=1e-12)
    s = (amax / FP8_MAX).to(torch.float32)
    q = (blk / s[..., :, None, :, None]).reshape(*lead, Nb * bn, Kb * bk)[..., :N, :K]
    return q.to(torch.float8_e4m3fn).contiguous(), s


def expand_block_scale(s: torch.Tensor, N: int, K: int, bn: int = BLOCK, bk: int = BLOCK) -> torch.Tensor:
    """[..., Nb, Kb] -> [..., N, K] (tests/test_fp8_blockscale_gemm.py:31-36)."""
    return s.repeat_interleave(bn, -2)[..., :N, :].repeat_interleave(bk, -1)[..., :K]


def dequant_block(wq: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    N, K = wq.shape[-2:]
    return decode(wq) * expand_block_scale(s, N, K)


def quantize_act_1x128(x: torch.Tensor):
    """Per token, per 128 columns: s = max(amax, 1e-12)/448 (fp32), q = (x / s).to(e4m3)."""
    M, K = x.shape
    g = x.float().reshape(M, K // BLOCK, BLOCK)
    s = (g.abs().amax(dim=-1).clamp(min=1e-12) / FP8_MAX).to(torch.float32)
    q = (g / s[:, :, None]).to(torch.float8_e4m3fn).reshape(M, K)
    return q, s


def dequant_act_1x128(xq: torch.Tensor, xs: torch.Tensor) -> torch.Tensor:
    return decode(xq) * xs.repeat_interleave(BLOCK, dim=1)


def linear_channel(x, wq, s, e5m2=False):
    """Y = X.float() @ (decode(Wq) * s[:, None]).T  (fp32)."""
    return x.float() @ (decode(wq, e5m2) * s.float().reshape(-1, 1)).T


def linear_tensor(x, wq, s, e5m2=False):
    return x.float() @ (decode(wq, e5m2) * s.float().reshape(())).T


def linear_block_w8a16(x, wq, ws):
    """The reference's block path keeps the activation in 16 bit (vllm/patches/vllm_for_multi_arc.patch:2671-2683)."""
    return x.float() @ dequant_block(wq, ws).T


def linear_block_w8a8(xq, xs, wq, ws):
    """dq(Aq, As) @ dq(Wq, Ws).T in fp32."""
    return dequant_act_1x128(xq, xs) @ dequant_block(wq, ws).T
