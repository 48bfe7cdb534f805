"""GPU parity at the FULL sizes of the five benchmark configurations: the launches the benchmark times.

The problems are generated on the device (seeded), run through the torch ops (C ABI underneath), and checked
against the CPU oracle on seeded slices of the output (oracle/slices.py): an output element of a linear layer
depends on one activation row and one weight row only and a MoE output row on one token only, so a slice of
the oracle is exact.  The selections take at least one column out of every 128-row weight strip and one token
out of every token tile, so every CTA of a launch contributes.  Gate: max|err| / max|ref| <= 1e-2
(16-bit output of an fp32 accumulation).  Kernel overlap mode 2 (weights static) is set as in the benchmark.
"""
import pytest
import torch

from gpu_util import DEV
from oracle import configs, fp8, int4, slices

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def e(lib_built):
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    import custom_esimd_kernels_vllm as pkg
    pkg.set_overlap_mode(2)
    yield pkg
    pkg.set_overlap_mode(1)
    torch.cuda.empty_cache()


def _gate(err, what, tol=TOL):
    assert err["max_rel_err"] <= tol and err["mean_rel_err"] <= tol and err["cos"] > 0.9999, (what, err)


def _int4_dev(N, K, seed, lead=()):
    g = torch.Generator(device=DEV).manual_seed(seed)
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, (*lead, N, K // 8), generator=g, device=DEV, dtype=torch.int32)
    s = (0.002 + torch.randn(*lead, N, K // 128, generator=g, device=DEV).abs() * 0.01).to(torch.bfloat16)
    return w, s


# ------------------------------------------------------------------ config 2: FP8 per-channel GEMV sweep, [27648, 5120]
@pytest.fixture(scope="module")
def c2_full():
    return configs.c2(seed=0, M=32)            # generated on the CPU exactly as the configuration states it


@pytest.mark.parametrize("M", [1, 8, 32])
def test_c2_fp8_channel_gemv_full_size(e, c2_full, M):
    wq, s = c2_full["wq"], c2_full["scale"]
    x = c2_full["x"][:M].contiguous()
    out = torch.empty(M, 27648, dtype=torch.bfloat16, device=DEV)
    wd, sd = wq.to(DEV), s.to(DEV)
    for _ in range(2):                          # the second launch overlaps the tail of the first (mode 2)
        e.esimd_gemv_fp8_pern(x.to(DEV), wd, sd, out, 27648, 5120)
    assert e.last_kernel() == "umma_w8_direct"
    ref = fp8.linear_channel(x, wq, s)          # every output column, on the CPU
    _gate(slices.errors(out, ref.to(torch.bfloat16)), f"C2 M={M}")
    assert e._lib.device_status() == 0


# ------------------------------------------------------------------ config 3: FP8 128x128 block GEMM, [4096 x 17408 x 5120]
@pytest.fixture(scope="module")
def c3_full(e):
    M, N, K = 4096, 17408, 5120
    g = torch.Generator(device=DEV).manual_seed(3)
    w = (torch.randn(N, K, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    wq, ws = e._impl.quantize_fp8(w, e._lib.SCALE_BLOCK128)       # bit-identical to oracle.fp8.quantize_block (own test)
    x = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
    del w
    toks = slices.pick(M, 24, 31, every=128)     # one token out of every 128-token tile, plus 24 more
    cols = slices.pick(N, 64, 32, every=128)     # one column out of every 128-row weight strip, plus 64 more
    return {"x": x, "wq": wq, "ws": ws, "toks": toks, "cols": cols}


def test_c3_fp8_block_w8a16_full_size(e, c3_full):
    c = c3_full
    out = torch.empty(4096, 17408, dtype=torch.bfloat16, device=DEV)
    e.esimd_gemm_fp8_blockscale(c["x"], c["wq"], c["ws"], out, 128, 128)
    all_t, all_c = torch.arange(4096), torch.arange(17408)
    _gate(slices.fp8_block_w8a16(c["x"], c["wq"], c["ws"], out, all_c, c["toks"]), "C3 w8a16, token slice x all columns")
    _gate(slices.fp8_block_w8a16(c["x"], c["wq"], c["ws"], out, c["cols"], all_t), "C3 w8a16, all tokens x column slice")
    assert e._lib.device_status() == 0


def test_c3_fp8_block_w8a8_full_size(e, c3_full):
    c = c3_full
    xq, xs = e.act_quant_fp8_1x128(c["x"])
    rq, rs = fp8.quantize_act_1x128(c["x"][c["toks"].to(DEV)].cpu())
    assert torch.equal(xq[c["toks"].to(DEV)].cpu().view(torch.uint8), rq.view(torch.uint8)), "activation codes differ from the oracle"
    assert torch.equal(xs[c["toks"].to(DEV)].cpu(), rs), "activation scales differ from the oracle"
    out = torch.empty(4096, 17408, dtype=torch.bfloat16, device=DEV)
    e.gemm_fp8_block_w8a8(xq, xs, c["wq"], c["ws"], out)
    all_t, all_c = torch.arange(4096), torch.arange(17408)
    _gate(slices.fp8_block_w8a8(xq, xs, c["wq"], c["ws"], out, all_c, c["toks"]), "C3 w8a8, token slice x all columns")
    _gate(slices.fp8_block_w8a8(xq, xs, c["wq"], c["ws"], out, c["cols"], all_t), "C3 w8a8, all tokens x column slice")
    assert e._lib.device_status() == 0


# ------------------------------------------------------------------ config 4: INT4 MoE, T=4096, E=128, top-8, H=2048, I=768
def test_c4_moe_int4_full_size(e):
    T, E, H, I, k = 4096, 128, 2048, 768, 8
    w13, s13 = _int4_dev(2 * I, H, 41, lead=(E,))
    w2, s2 = _int4_dev(H, I, 42, lead=(E,))
    g = torch.Generator(device=DEV).manual_seed(43)
    x = torch.randn(T, H, generator=g, device=DEV).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=DEV).to(torch.bfloat16)
    toks = slices.pick(T, 192, 44)
    experts = (slices.LazyExperts(w13, s13, torch.bfloat16), slices.LazyExperts(w2, s2, torch.bfloat16))   # shared by both routes
    out = e.moe_prefill_full_int4(x, logits, w13, s13, w2, s2, k, E)
    err = slices.moe_int4(x, logits, w13, s13, w2, s2, k, out, toks, experts)
    # the same pipeline with the weights rounded to the activation type exactly as the oracle rounds them
    # (no activation pre-pass): separates the kernels' arithmetic from the oracle's bf16 weight rounding
    e.set_force_kernel(3)
    try:
        out_exact = e.moe_prefill_full_int4(x, logits, w13, s13, w2, s2, k, E)
    finally:
        e.set_force_kernel(0)
    err_exact = slices.moe_int4(x, logits, w13, s13, w2, s2, k, out_exact, toks, experts)
    print("C4 pipeline vs oracle: default route %s ; exact-weight route %s" % (err, err_exact))
    _gate(err_exact, "C4 exact-weight route")
    _gate(err, "C4 default route")
    assert e._lib.device_status() == 0


# ------------------------------------------------------------------ config 5: Llama-70B-shape INT4 linears at M = 64 and M = 2048
@pytest.mark.parametrize("M", [64, 2048])
@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
def test_c5_int4_linear_full_size(e, name, M):
    N, K = configs.C5_LAYER[name]
    w, s = _int4_dev(N, K, 50 + len(name))
    x = torch.randn(M, K, generator=torch.Generator(device=DEV).manual_seed(M), device=DEV).to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    e.esimd_gemm_int4_pgrp(x, w, s, out)
    cols = slices.pick(N, 128, 51, every=128)
    toks = torch.arange(M) if M <= 64 else slices.pick(M, 32, 52, every=256)
    _gate(slices.int4_linear(x, w, s, out, cols, toks), f"C5 {name} M={M}, token slice x column slice")
    if M > 64:
        _gate(slices.int4_linear(x, w, s, out, slices.pick(N, 48, 53), torch.arange(M)), f"C5 {name} M={M}, all tokens")
    assert e._lib.device_status() == 0


# ------------------------------------------------------------------ INT4 scales outside fp16's normal range
@pytest.mark.parametrize("scale_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("magnitude", [1e-5, 1e-8, 3e4])
def test_int4_scales_outside_fp16_range(e, scale_dtype, magnitude):
    """The tensor-core route forms (q - 8) * scale in fp16; scales far below fp16's smallest normal (6.1e-5) or so
    large that 8 * scale overflows it must still give the oracle's result (a power of two per output row keeps the
    fp16 operand in range)."""
    N, K, M = 512, 1024, 64
    g = torch.Generator().manual_seed(int(magnitude * 1e9) % 1000 + 1)
    q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
    s = ((0.2 + torch.rand(N, K // 128, generator=g)) * magnitude).to(scale_dtype)
    s[::7] *= 64.0                                               # rows of different magnitude in one strip
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    e.esimd_gemm_int4_pgrp(x.to(DEV), int4.pack_nmajor_i32(q).to(DEV), s.to(DEV), out)
    assert e.last_kernel() == "umma_wo"
    ref = x.float() @ ((q.float() - 8.0) * s.float().repeat_interleave(128, dim=1)).T       # unrounded weights
    _gate(slices.errors(out, ref.to(torch.bfloat16)), f"scales ~{magnitude} {scale_dtype}")
