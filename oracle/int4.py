"""INT4 (symmetric, zero-point 8, group 128) formats: quantisers, packers, dequant, linear."""
import numpy as np
import torch

GROUP = 128
MARLIN_SHUFFLE = (0, 4, 1, 5, 2, 6, 3, 7)     # tests/test_moe_int4_kernel.py:86-104
MARLIN_UNSHUFFLE = (0, 2, 4, 6, 1, 3, 5, 7)   # csrc/moe_prefill/moe_prefill_int4.sycl:136


def quantize_ggml_q4_0(w: torch.Tensor, group: int = GROUP):
    """GGML q4_0: scale = signed_max / -8 (may be negative), q = clamp(int(w/scale + 8.5), 0, 15).

    Follows tests/test_gemv_int4.py:118-169.  Returns (q uint8 [N, K] in 0..15, scale fp16 [N, K/group]).
    """
    N, K = w.shape
    g = w.float().reshape(N, K // group, group)
    _, idx = g.abs().max(dim=-1, keepdim=True)
    signed_max = g.gather(-1, idx)
    scale = (signed_max / -8.0).squeeze(-1).to(torch.float16)
    se = scale.float().unsqueeze(-1)
    inv = torch.where(se.abs() > 1e-10, 1.0 / se, torch.zeros_like(se))
    q = (g * inv + 8.5).to(torch.int32).clamp(0, 15).reshape(N, K)
    return q.to(torch.uint8), scale


def quantize_q4_0_device(w: torch.Tensor, group: int = GROUP):
    """The on-device GGML Q4_0 quantiser, operation by operation (csrc/xpu/q4_0_quant.sycl:60-104).

    Differs from quantize_ggml_q4_0 (the tests' Python quantiser) in two places: the inverse is taken of the fp32
    scale, not of its fp16 rounding, and when +amax and -amax both occur the positive one is the signed maximum.
    Returns (q uint8 [N, K] in 0..15, scale fp16 [N, K/group]).
    """
    N, K = w.shape
    g = w.float().reshape(N, K // group, group)
    max_pos = g.amax(dim=-1)
    neg_max = (-g).amax(dim=-1)
    max_signed = torch.where(max_pos >= neg_max, max_pos, -neg_max)
    d = max_signed / -8.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    biased = g * inv.unsqueeze(-1) + 8.5                      # product and sum rounded separately (fp32 tensors)
    q = biased.to(torch.int32).clamp(0, 15).reshape(N, K)     # conversion truncates
    return q.to(torch.uint8), d.to(torch.float16)


def quantize_symmetric(w: torch.Tensor, group: int = GROUP, scale_dtype=torch.float16):
    """amax/7 symmetric quantiser: q = round(w / scale).clip(-8, 7) + 8.

    Follows tests/test_moe_int4_kernel.py:42-65 (numpy round = half to even).
    """
    N, K = w.shape
    g = w.float().numpy().reshape(N, K // group, group)
    amax = np.abs(g).max(axis=2)
    scale = np.where(amax > 0, amax / 7.0, 1.0).astype(np.float16)
    q = np.round(g / scale[:, :, None].astype(np.float32)).clip(-8, 7).astype(np.int32) + 8
    return torch.from_numpy(q.reshape(N, K).astype(np.uint8)), torch.from_numpy(scale).to(scale_dtype)


# ---------------------------------------------------------------- packers
def pack_nmajor_u8(q: torch.Tensor) -> torch.Tensor:
    """[N, K] nibbles -> uint8 [N, K/2], low nibble = even k (tests/test_gemv_int4.py:163-167)."""
    q = q.to(torch.uint8)
    return ((q[..., 0::2] & 0xF) | ((q[..., 1::2] & 0xF) << 4)).contiguous()


def pack_nmajor_i32(q: torch.Tensor) -> torch.Tensor:
    """[..., N, K] nibbles -> int32 [..., N, K/8], nibble i at bits 4i (tests/test_moe_int4_kernel.py:57-61)."""
    qq = q.to(torch.int64).reshape(*q.shape[:-1], q.shape[-1] // 8, 8)
    out = torch.zeros(qq.shape[:-1], dtype=torch.int64)
    for b in range(8):
        out |= (qq[..., b] & 0xF) << (4 * b)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32).contiguous()


def unpack_nmajor_i32(w: torch.Tensor) -> torch.Tensor:
    """int32 [..., N, K/8] -> nibbles uint8 [..., N, K] (tests/test_moe_int4_kernel.py:74-77)."""
    u = w.to(torch.int64) & 0xFFFFFFFF
    sh = torch.arange(8, dtype=torch.int64) * 4
    nib = (u.unsqueeze(-1) >> sh) & 0xF
    return nib.reshape(*w.shape[:-1], w.shape[-1] * 8).to(torch.uint8)


def unpack_nmajor_u8(w: torch.Tensor) -> torch.Tensor:
    """uint8 [..., N, K/2] -> nibbles [..., N, K] (tests/test_gemv_int4.py:193-204)."""
    lo = w & 0xF
    hi = (w >> 4) & 0xF
    return torch.stack([lo, hi], dim=-1).reshape(*w.shape[:-1], w.shape[-1] * 2)


def marlin_shuffle_words(words: torch.Tensor) -> torch.Tensor:
    """Reorder the eight nibbles of each int32: new[p] = old[MARLIN_SHUFFLE[p]] (tests/test_moe_int4_kernel.py:86-104)."""
    u = words.to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros_like(u)
    for new_pos, old_pos in enumerate(MARLIN_SHUFFLE):
        out |= ((u >> (4 * old_pos)) & 0xF) << (4 * new_pos)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def to_kmajor(w_nmajor_i32: torch.Tensor, scale_nmajor: torch.Tensor, marlin: bool):
    """N-major int32 [..., N, K/8] + scales [..., N, K/g] -> K-major [..., K/8, N] (+ marlin shuffle), scales [..., K/g, N].

    Follows ipex_transform_expert_weights, tests/test_moe_int4_kernel.py:107-125; without the
    shuffle it is the materialised GPTQ view of vllm/patches/vllm_for_multi_arc.patch:5519-5526.
    """
    wt = w_nmajor_i32.transpose(-1, -2).contiguous()
    st = scale_nmajor.transpose(-1, -2).contiguous()
    if marlin:
        wt = marlin_shuffle_words(wt)
    return wt, st


def unpack_kmajor(w: torch.Tensor, marlin: bool) -> torch.Tensor:
    """K-major int32 [..., K/8, N] -> nibbles [..., N, K]."""
    u = w.to(torch.int64) & 0xFFFFFFFF
    K8, N = w.shape[-2], w.shape[-1]
    out = torch.empty(*w.shape[:-2], N, K8 * 8, dtype=torch.uint8)
    for j in range(8):
        slot = MARLIN_UNSHUFFLE[j] if marlin else j
        out[..., j::8] = ((u >> (4 * slot)) & 0xF).transpose(-1, -2).to(torch.uint8)
    return out


def u4_to_s4_bytes(w_u8: torch.Tensor) -> torch.Tensor:
    """uint4 bytes -> two's-complement int4 bytes (value = u4 - 8), tests/test_cutlass_nmajor_int4_pack.py:56-75."""
    lo = (w_u8 & 0xF).to(torch.int16) - 8
    hi = ((w_u8 >> 4) & 0xF).to(torch.int16) - 8
    return ((lo & 0xF) | ((hi & 0xF) << 4)).to(torch.uint8)


def unpack_s4_bytes(w_s4: torch.Tensor) -> torch.Tensor:
    """two's-complement nibbles -> signed values int8 [..., N, K] (csrc/moe_batch/int4_nmajor_gemm.h:137)."""
    nib = unpack_nmajor_u8(w_s4).to(torch.int16)
    return torch.where(nib >= 8, nib - 16, nib).to(torch.int8)


# ---------------------------------------------------------------- dequant + linear
def dequant(q: torch.Tensor, scale: torch.Tensor, dtype, group: int = GROUP) -> torch.Tensor:
    """(q - 8) * scale, one rounding to dtype.  q: nibbles [..., N, K]; scale [..., N, K/group].

    tests/test_gemv_int4.py:172-210, tests/test_moe_int4_kernel.py:68-83.
    """
    v = q.to(torch.float32) - 8.0
    s = scale.float().repeat_interleave(group, dim=-1)
    return (v * s).to(dtype)


def dequant_signed(v: torch.Tensor, scale: torch.Tensor, dtype, group: int = GROUP) -> torch.Tensor:
    s = scale.float().repeat_interleave(group, dim=-1)
    return (v.to(torch.float32) * s).to(dtype)


def linear(x: torch.Tensor, q: torch.Tensor, scale: torch.Tensor, group: int = GROUP) -> torch.Tensor:
    """Y = X.float() @ dequant(W).float().T in fp32 (tests/test_gemv_int4.py:213-233). Returns fp32."""
    wd = dequant(q, scale, x.dtype, group)
    return x.float() @ wd.float().T
