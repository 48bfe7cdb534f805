"""GPU parity of the dense ops against the CPU oracle, called through the torch custom ops (which
bind the C ABI).  Tolerance: max|err| / max|ref| <= 1e-2 for 16-bit outputs of an fp32 accumulation;
dequantised weights are compared bit for bit."""
import numpy as np
import pytest
import torch

from gpu_util import DEV, assert_close
from oracle import configs, fp8, int4

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def e(lib_built):
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    import custom_esimd_kernels_vllm as pkg
    assert pkg._lib.lib.b2q_device_ok() == 0, "libb2q.so targets sm_100a only"
    return pkg


def _rand_int4(N, K, dtype, seed, neg_scales=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
    s = 0.002 + torch.randn(N, K // 128, generator=g).abs() * 0.01
    if neg_scales:
        s = s * torch.where(torch.rand(N, K // 128, generator=g) < 0.5, -1.0, 1.0)
    return q, s.to(dtype)


# ------------------------------------------------------------------ dequant: bit-exact gate
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_dequant_int4_all_layouts_bit_exact(e, dtype):
    q, s = _rand_int4(80, 384, torch.bfloat16 if dtype != torch.float16 else torch.float16, 3, neg_scales=True)
    ref = int4.dequant(q, s, dtype)
    w32 = int4.pack_nmajor_i32(q)
    L = e._lib
    out = e.dequant_int4(w32.to(DEV), s.to(DEV), dtype, L.W4_NMAJOR)
    assert torch.equal(out.cpu(), ref)
    out = e.dequant_int4(int4.pack_nmajor_u8(q).to(DEV), s.to(DEV), dtype, L.W4_NMAJOR)
    assert torch.equal(out.cpu(), ref)
    for marlin, lay in ((False, L.W4_KMAJOR), (True, L.W4_KMAJOR_MARLIN)):
        wk, sk = int4.to_kmajor(w32, s, marlin)
        out = e.dequant_int4(wk.to(DEV), sk.to(DEV), dtype, lay)
        assert torch.equal(out.cpu(), ref), lay
    s4 = int4.u4_to_s4_bytes(int4.pack_nmajor_u8(q))
    out = e.dequant_int4(s4.to(DEV), s.to(DEV), dtype, L.W4_NMAJOR_S4)
    assert torch.equal(out.cpu(), ref)


def test_dequant_int4_golden(e, golden):
    g = golden("int4_ggml")
    out = e.dequant_int4(torch.from_numpy(g["packed"]).to(DEV), torch.from_numpy(g["scale"]).to(DEV), torch.float16)
    assert torch.equal(out.cpu(), torch.from_numpy(g["deq"]))
    g = golden("int4_sym")
    out = e.dequant_int4(torch.from_numpy(g["ipex_q"][0]).to(DEV), torch.from_numpy(g["ipex_s"][0]).to(DEV),
                         torch.float16, e._lib.W4_KMAJOR_MARLIN)
    assert torch.equal(out.cpu(), torch.from_numpy(g["deq"]))


def test_dequant_fp8_every_code_exact(e, golden):
    codes = torch.arange(256, dtype=torch.uint8).repeat(8, 1).contiguous()          # [8, 256]
    ones = torch.ones(8, dtype=torch.float32)
    for fmt_dtype, key in ((torch.float8_e4m3fn, "e4m3_codes"), (torch.float8_e5m2, "e5m2_codes")):
        out = e.dequant_fp8(codes.view(fmt_dtype).to(DEV), ones.to(DEV), e._lib.SCALE_CHANNEL, torch.float32).cpu()
        ref = torch.from_numpy(golden("fp8_block")[key])
        fin = torch.isfinite(ref)
        assert torch.equal(out[0][fin], ref[fin])
        assert torch.equal(torch.isnan(out[0]), torch.isnan(ref))
    g = golden("fp8_block")
    out = e.dequant_fp8(torch.from_numpy(g["wq"]).to(DEV), torch.from_numpy(g["ws"]).to(DEV), e._lib.SCALE_BLOCK128,
                        torch.float32)
    assert torch.equal(out.cpu(), torch.from_numpy(g["wd"]))


# ------------------------------------------------------------------ INT4 linear
INT4_SHAPES = [(2560, 2048), (2048, 512), (3072, 2048), (16, 2048), (512, 2048), (128, 7168), (256, 14336), (1024, 128),
               (1000, 384)]


@pytest.mark.parametrize("N,K", INT4_SHAPES)
@pytest.mark.parametrize("M", [1, 7, 16, 33, 64])
def test_int4_linear_shapes(e, N, K, M):
    dtype = torch.bfloat16 if (N + M) % 2 == 0 else torch.float16
    q, s = _rand_int4(N, K, dtype, N + K + M, neg_scales=True)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(dtype)
    ref = int4.linear(x, q, s)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    op = e.esimd_gemv_int4 if M == 1 else e.esimd_gemm_int4_pgrp
    r = op(x.to(DEV), int4.pack_nmajor_u8(q).to(DEV), s.to(DEV), out)
    assert r.data_ptr() == out.data_ptr()
    assert_close(out, ref, what=f"int4 M={M} N={N} K={K}")


def test_int4_config1_all_presentations(e):
    c = configs.c1()
    ref = int4.linear(c["x"], c["q"], c["scale"])
    x = c["x"].to(DEV)
    w32 = c["w_i32"].to(DEV)
    s = c["scale"].to(DEV)
    for w, sc in ((w32, s), (w32.view(torch.uint8), s), (w32.t(), s.t().contiguous())):
        out = torch.empty(16, 4096, dtype=torch.bfloat16, device=DEV)
        e.esimd_gemm_int4_pgrp(x, w, sc, out)
        assert_close(out, ref, what="C1")


def test_int4_golden_gemv(e, golden):
    g = golden("int4_ggml")
    x = torch.from_numpy(g["x"]).to(DEV)
    out = torch.empty(1, 24, dtype=torch.float16, device=DEV)
    e.esimd_gemv_int4(x, torch.from_numpy(g["packed"]).to(DEV), torch.from_numpy(g["scale"]).to(DEV), out)
    assert_close(out, torch.from_numpy(g["y"]), what="golden gemv")


def test_int4_fused2_and_s4(e):
    q0, s0 = _rand_int4(256, 512, torch.bfloat16, 1)
    q1, s1 = _rand_int4(64, 512, torch.bfloat16, 2)
    x = torch.randn(1, 512).to(torch.bfloat16)
    o0 = torch.empty(1, 256, dtype=torch.bfloat16, device=DEV)
    o1 = torch.empty(1, 64, dtype=torch.bfloat16, device=DEV)
    r = e.esimd_gemv_int4_fused2(x.to(DEV), int4.pack_nmajor_u8(q0).to(DEV), s0.to(DEV), o0,
                                 int4.pack_nmajor_u8(q1).to(DEV), s1.to(DEV), o1)
    assert r.data_ptr() == o0.data_ptr()
    assert_close(o0, int4.linear(x, q0, s0), what="fused2/0")
    assert_close(o1, int4.linear(x, q1, s1), what="fused2/1")


def test_int4_rejects_bad_arguments(e):
    x = torch.zeros(2, 256, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(16, 128, dtype=torch.uint8, device=DEV)
    s = torch.zeros(16, 2, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError):
        e.esimd_gemm_int4_pgrp(x, w, s, torch.zeros(2, 8, dtype=torch.bfloat16, device=DEV))      # wrong N
    with pytest.raises(RuntimeError):
        e.esimd_gemm_int4_pgrp(x, w, s, torch.zeros(2, 16, dtype=torch.float16, device=DEV))      # dtype mismatch
    with pytest.raises(RuntimeError):
        e.esimd_gemm_int4_pgrp(x.float(), w, s, torch.zeros(2, 16, dtype=torch.float32, device=DEV))


# ------------------------------------------------------------------ FP8 linear
@pytest.mark.parametrize("M", [1, 8, 32])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fp8_per_channel(e, M, dtype):
    c = configs.c2(seed=M, M=M, N=1536, K=5120, dtype=dtype)
    ref = fp8.linear_channel(c["x"], c["wq"], c["scale"])
    out = torch.empty(M, 1536, dtype=dtype, device=DEV)
    for sdt in (torch.float32, torch.float16):
        e.esimd_gemv_fp8_pern(c["x"].to(DEV), c["wq"].to(DEV), c["scale"].to(sdt).to(DEV), out, 1536, 5120)
        ref_s = fp8.linear_channel(c["x"], c["wq"], c["scale"].to(sdt))
        assert_close(out, ref_s, what=f"fp8 pern M={M} {dtype} scale {sdt}")


@pytest.mark.parametrize("M,N,K", [(1, 1024, 5120), (3, 1000, 1056), (64, 512, 2048), (128, 256, 1024)])
def test_fp8_per_tensor_and_e5m2(e, M, N, K):
    g = torch.Generator().manual_seed(M + N)
    w = torch.randn(N, K, generator=g) * 0.05
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    wq, s = fp8.quantize_tensor(w)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    e.esimd_gemm_fp8_pert(x.to(DEV), wq.to(DEV), s.to(DEV), out)
    assert_close(out, fp8.linear_tensor(x, wq, s), what="fp8 pert e4m3")
    w5 = (w / s).to(torch.float8_e5m2)
    e.esimd_gemv_fp8_pert(x.to(DEV), w5.to(DEV), s.to(DEV), out)
    assert_close(out, fp8.linear_tensor(x, w5, s, e5m2=True), what="fp8 pert e5m2")


@pytest.mark.parametrize("M,N,K", [(1, 1024, 5120), (1, 5120, 6144), (2, 5120, 5120), (7, 5120, 5120), (9, 5120, 5120),
                                   (12, 5120, 5120), (33, 5120, 5120), (64, 5120, 5120), (1, 1000, 5120),
                                   (4, 1000, 5120)])
def test_fp8_blockscale_w8a16(e, M, N, K):
    g = torch.Generator().manual_seed(1234 + M * 131 + N + K)
    w = torch.randn(N, K, generator=g) * 0.3
    wq, ws = fp8.quantize_block(w)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.float16)
    out = torch.empty(M, N, dtype=torch.float16, device=DEV)
    e.esimd_gemm_fp8_blockscale(a.to(DEV), wq.to(DEV), ws.to(DEV), out, 128, 128)
    assert_close(out, fp8.linear_block_w8a16(a, wq, ws), what=f"fp8 block M={M} N={N} K={K}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fp8_all_finite_codes_through_gemm_are_exact(e, dtype):
    """Every raw e4m3 code times x = 1 over K = 128: the result is 128 * decode(code), exactly."""
    raw = torch.arange(256, dtype=torch.uint8).view(256, 1).expand(256, 128).contiguous()
    reference = torch.from_numpy(fp8.e4m3_table()) * 128
    finite = torch.isfinite(reference)
    x = torch.ones(1, 128, dtype=dtype, device=DEV)
    scale = torch.ones(2, 1, dtype=torch.float32, device=DEV)
    out = torch.empty(1, 256, dtype=dtype, device=DEV)
    e.esimd_gemm_fp8_blockscale(x, raw.to(DEV), scale, out, 128, 128)
    got = out[0].float().cpu()
    exp = reference.to(dtype).float()
    assert torch.equal(got[finite], exp[finite])
    assert got[0x80] == 0.0
    ones = torch.ones(256, dtype=torch.float32, device=DEV)
    e.esimd_gemv_fp8_pern(x, raw.to(DEV), ones, out, 256, 128)
    assert torch.equal(out[0].float().cpu()[finite], exp[finite])


def test_act_quant_1x128_bit_exact(e):
    x = torch.randn(37, 512, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    x[3, 128:256] = 0
    xq, xs = e.act_quant_fp8_1x128(x.to(DEV))
    rq, rs = fp8.quantize_act_1x128(x)
    assert torch.equal(xs.cpu(), rs)
    assert torch.equal(xq.cpu().view(torch.uint8), rq.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 8, 33, 64])
def test_fp8_decode_path_keeps_activations_exact(e, M, dtype):
    """Decode shapes run on the 8-bit MMA with the activations split into e4m3 terms.  With an identity weight
    (code 0x38 = 1.0 on the diagonal) and unit scales the output must equal the activations bit for bit, for every
    mantissa pattern and over twelve binades of dynamic range inside one row."""
    K = N = 256
    g = torch.Generator().manual_seed(17 + M)
    mant = torch.rand(M, K, generator=g) + 1.0
    expo = torch.randint(-6, 6, (M, K), generator=g).float()
    sign = torch.where(torch.rand(M, K, generator=g) < 0.5, -1.0, 1.0)
    x = (sign * mant * torch.exp2(expo)).to(dtype)
    x[:, 5] = 0
    w = torch.zeros(N, K, dtype=torch.uint8)
    w[torch.arange(N), torch.arange(K)] = 0x38
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    e.esimd_gemv_fp8_pern(x.to(DEV), w.to(DEV), torch.ones(N, device=DEV), out, N, K)
    assert e.last_kernel() == "umma_w8_direct"
    assert torch.equal(out.cpu(), x)


def test_fp8_decode_path_outliers_and_strip_heights(e):
    """Rows with a 10^4 outlier, N values that make the launch pick strips lower than 128 rows or cut strips
    along k, and a K that is not a multiple of 128."""
    for M, N, K in ((4, 27648 // 8 + 24, 1088), (16, 148 * 96 + 8, 512), (2, 640, 2112), (48, 9000, 256)):
        g = torch.Generator().manual_seed(N + K)
        w = torch.randn(N, K, generator=g) * 0.05
        wq, s = fp8.quantize_channel(w)
        x = torch.randn(M, K, generator=g)
        x[:, 7] *= 1e4
        x = x.to(torch.bfloat16)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        e.esimd_gemv_fp8_pern(x.to(DEV), wq.to(DEV), s.to(DEV), out, N, K)
        assert e.last_kernel() == "umma_w8_direct"
        assert_close(out, fp8.linear_channel(x, wq, s), what=f"fp8 decode M={M} N={N} K={K}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K", [(1, 128), (4, 256), (16, 128), (256, 512), (1024, 2048), (512, 5120)])
def test_q4_0_quantize_bit_exact(e, M, K, dtype):
    """On-device GGML Q4_0 quantiser (shapes of tests/test_q4_0_quant_xpu.py:52-61): words and scales equal the
    restated kernel arithmetic bit for bit, including groups that hold +amax and -amax, all-zero groups and
    values that land exactly on a rounding boundary."""
    torch.manual_seed(M * 7 + K)
    x = (torch.randn(M, K) * 0.5).to(dtype)
    x[0, :128] = 0
    if M > 1:
        x[1, 5], x[1, 77] = 1.5, -1.5          # tie of magnitudes: the positive one is the signed maximum
        x[1, 6] = 1.5 * 0.3125                 # 2.5 steps: exactly between two codes
    q = torch.empty(M, K // 8, dtype=torch.int32, device=DEV)
    s = torch.empty(M, K // 128, dtype=torch.float16, device=DEV)
    torch.ops.custom_esimd_kernels_vllm.q4_0_quantize(x.to(DEV), q, s)
    rq, rs = int4.quantize_q4_0_device(x)
    assert torch.equal(s.cpu().view(torch.int16), rs.view(torch.int16))
    assert torch.equal(q.cpu(), int4.pack_nmajor_i32(rq).to(torch.int32))
    # what it produces is what the INT4 linear consumes
    if M >= 16:
        a = torch.randn(4, K).to(dtype)
        out = torch.empty(4, M, dtype=dtype, device=DEV)
        e.esimd_gemm_int4_pgrp(a.to(DEV), q, s.to(dtype), out)
        assert_close(out, int4.linear(a, rq, rs.to(dtype)), what="linear on device-quantised weights")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,K", [(16, 128), (256, 512), (512, 2048), (128, 4096), (256, 3072)])
def test_resadd_norm_gemv_fused_ops(e, N, K, dtype):
    """esimd_resadd_norm_gemv_{int4,fp8}_pert and the two-matrix variant (shapes of tests/test_resadd_norm_gemv_int4.py:62-69):
    residual updated in place, normed_out and the GEMV outputs against the step-by-step oracle."""
    from oracle import fused
    g = torch.Generator().manual_seed(42 + N)
    hidden = torch.randn(1, K, generator=g).to(dtype)
    residual = torch.randn(1, K, generator=g).to(dtype)
    nw = (torch.randn(K, generator=g) * 0.1 + 1.0).to(dtype)
    ref_res, ref_normed = fused.resadd_rmsnorm(hidden, residual, nw, 1e-6)
    # INT4
    q, s = _rand_int4(N, K, dtype, N + K)
    res_d, normed_d = residual.to(DEV).clone(), torch.empty(1, K, dtype=dtype, device=DEV)
    out = torch.empty(1, N, dtype=dtype, device=DEV)
    r = e.esimd_resadd_norm_gemv_int4_pert(hidden.to(DEV), res_d, nw.to(DEV), int4.pack_nmajor_i32(q).to(DEV), s.to(DEV), out, normed_d, 1e-6)
    assert r.data_ptr() == out.data_ptr()
    assert torch.equal(res_d.cpu(), ref_res), "residual update must be the rounded fp32 sum"
    assert_close(normed_d, ref_normed, what="normed_out", tol=4e-3)      # one ulp of the 16-bit type around rsqrt differences
    assert_close(out, int4.linear(normed_d.cpu(), q, s), what=f"resadd+norm+int4 gemv N={N} K={K}")
    # FP8 per tensor, one and two matrices
    w = torch.randn(N, K, generator=g) * 0.05
    wq, ws = fp8.quantize_tensor(w)
    w2 = torch.randn(2 * N, K, generator=g) * 0.05
    wq2, ws2 = fp8.quantize_tensor(w2)
    res_d = residual.to(DEV).clone()
    normed_d.zero_()
    hd, nwd, wqd, wsd = hidden.to(DEV), nw.to(DEV), wq.to(DEV), ws.to(DEV)
    before = e.launch_count()
    e.esimd_resadd_norm_gemv_fp8_pert(hd, res_d, nwd, wqd, wsd, out, normed_d, 1e-6)
    assert e.launch_count() - before == 2, "the norm must run inside the GEMV's activation pre-pass: two launches in all"
    assert torch.equal(res_d.cpu(), ref_res)
    assert_close(normed_d, ref_normed, what="normed_out of the fused pre-pass", tol=4e-3)
    assert_close(out, fp8.linear_tensor(normed_d.cpu(), wq, ws), what="resadd+norm+fp8 gemv")
    res_d = residual.to(DEV).clone()
    o1 = torch.empty(1, 2 * N, dtype=dtype, device=DEV)
    e.esimd_resadd_norm_gemv2_fp8_pert(hidden.to(DEV), res_d, nw.to(DEV), wq.to(DEV), ws.to(DEV), out, wq2.to(DEV), ws2.to(DEV), o1, 1e-6)
    assert torch.equal(res_d.cpu(), ref_res)
    assert_close(out, fp8.linear_tensor(normed_d.cpu(), wq, ws), what="gemv2 / 0")
    assert_close(o1, fp8.linear_tensor(normed_d.cpu(), wq2, ws2), what="gemv2 / 1")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("HV,V,N", [(8, 128, 2048), (16, 128, 512), (4, 256, 1000)])
def test_gated_norm_gemv_fused_ops(e, HV, V, N, dtype):
    """esimd_norm_gemv_{fp8_pert, fp8_blockscale, int4_pert} (first shape: tests/test_fp8_blockscale_fusions.py:81-100)."""
    from oracle import fused
    g = torch.Generator().manual_seed(HV + V + N)
    core = (torch.randn(HV, V, generator=g) * 0.3).to(dtype)
    gate = (torch.randn(HV, V, generator=g) * 0.3).to(dtype)
    nw = (torch.randn(V, generator=g) * 0.1 + 1.0).to(dtype)
    K = HV * V
    normed = fused.gated_rmsnorm(core, gate, nw, 1e-6)
    got = e._impl.gated_rmsnorm(core.to(DEV), gate.to(DEV), nw.to(DEV), 1e-6)
    assert_close(got, normed, what="gated rmsnorm", tol=4e-3)
    normed_d = got.cpu()
    w = torch.randn(N, K, generator=g) * 0.2
    out = torch.empty(1, N, dtype=dtype, device=DEV)
    wq, ws = fp8.quantize_tensor(w)
    e.esimd_norm_gemv_fp8_pert(core.to(DEV), gate.to(DEV), nw.to(DEV), wq.to(DEV), ws.to(DEV), out, HV, V, 1e-6)
    assert_close(out, fp8.linear_tensor(normed_d, wq, ws), what="gated norm + fp8 pert")
    if N % 128 == 0:
        wqb, wsb = fp8.quantize_block(w)
        e.esimd_norm_gemv_fp8_blockscale(core.to(DEV), gate.to(DEV), nw.to(DEV), wqb.to(DEV), wsb.to(DEV), out, HV, V, 1e-6)
        assert_close(out, fp8.linear_block_w8a16(normed_d, wqb, wsb), what="gated norm + fp8 block")
    q, s = _rand_int4(N, K, dtype, N)
    e.esimd_norm_gemv_int4_pert(core.to(DEV), gate.to(DEV), nw.to(DEV), int4.pack_nmajor_i32(q).to(DEV), s.to(DEV), out, HV, V, 1e-6)
    assert_close(out, int4.linear(normed_d, q, s), what="gated norm + int4")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,K,scalar", [(256, 512, 0.5), (1024, 2816, 1.7), (128, 4096, 1.0)])
def test_scaled_resadd_norm_gemv_fp8(e, N, K, scalar, dtype):
    """esimd_scaled_resadd_norm_gemv_fp8_pert: residual <- (h + r) * scalar in place, then norm and the per-tensor GEMV."""
    from oracle import fused
    g = torch.Generator().manual_seed(N + K)
    hidden = torch.randn(1, K, generator=g).to(dtype)
    residual = torch.randn(1, K, generator=g).to(dtype)
    nw = (torch.randn(K, generator=g) * 0.1 + 1.0).to(dtype)
    wq, ws = fp8.quantize_tensor(torch.randn(N, K, generator=g) * 0.05)
    ref_res, ref_normed = fused.scaled_resadd_rmsnorm(hidden, residual, nw, 1e-6, scalar)
    res_d = residual.to(DEV).clone()
    out = torch.empty(1, N, dtype=dtype, device=DEV)
    r = e.esimd_scaled_resadd_norm_gemv_fp8_pert(hidden.to(DEV), res_d, nw.to(DEV), wq.to(DEV), ws.to(DEV), out, 1e-6, scalar)
    assert r is None
    assert torch.equal(res_d.cpu(), ref_res)
    assert_close(out, fp8.linear_tensor(ref_normed, wq, ws), what="scaled resadd + norm + fp8 gemv")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,K", [(128, 2816), (64, 512), (8, 1024)])
def test_norm_gemv_norm_two_outputs(e, N, K, dtype):
    """esimd_norm_gemv_norm_fp16: router logits and the MoE input from one shared 1/rms; the residual is not written."""
    from oracle import fused
    g = torch.Generator().manual_seed(N * K)
    residual = torch.randn(1, K, generator=g).to(dtype)
    sw = (torch.randn(K, generator=g) * 0.2 + 1.0).to(dtype)
    pw = (torch.randn(K, generator=g) * 0.2 + 1.0).to(dtype)
    proj = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
    ref_in, ref_moe = fused.norm_two_scales(residual, sw, pw, 1e-6)
    res_d = residual.to(DEV).clone()
    logits = torch.empty(1, N, dtype=dtype, device=DEV)
    moe_in = torch.empty(1, K, dtype=dtype, device=DEV)
    e.esimd_norm_gemv_norm_fp16(res_d, sw.to(DEV), proj.to(DEV), pw.to(DEV), logits, moe_in, 1e-6)
    assert torch.equal(res_d.cpu(), residual)
    assert_close(moe_in, ref_moe, what="moe_input", tol=4e-3)
    assert_close(logits, (ref_in.float() @ proj.float().T).to(dtype), what="router logits")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("N,K", [(256, 384), (300, 200), (1, 128), (129, 130), (1024, 5120)])
def test_fp8_weight_quantisers_bit_exact(e, N, K, dtype, golden):
    """b2q_quantize_fp8 in its three scale modes: scales and e4m3 codes identical to the oracle quantisers (which the
    golden vectors pin to the reference's block recipe), ragged edge blocks, an all-zero block and a strided source."""
    I_, L = e._impl, e._lib
    g = torch.Generator().manual_seed(N * 3 + K)
    w = (torch.randn(N, K, generator=g) * 0.07).to(dtype)
    if N > 128:
        w[128:, :min(K, 128)] = 0                      # a block of zeros: scale clamps at 1e-12 / 448
    for mode, ref in ((L.SCALE_BLOCK128, fp8.quantize_block), (L.SCALE_CHANNEL, fp8.quantize_channel),
                      (L.SCALE_TENSOR, fp8.quantize_tensor)):
        rq, rs = ref(w)
        q, s = I_.quantize_fp8(w.to(DEV), mode)
        assert torch.equal(s.cpu().reshape(rs.shape), rs), f"scale, mode {mode}"
        assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8)), f"codes, mode {mode}"
    wide = torch.zeros(N, K + 24, dtype=dtype)
    wide[:, :K] = w
    q2, s2 = I_.quantize_fp8(wide.to(DEV)[:, :K], L.SCALE_BLOCK128)
    rq, rs = fp8.quantize_block(w)
    assert torch.equal(s2.cpu(), rs) and torch.equal(q2.cpu().view(torch.uint8), rq.view(torch.uint8))
    if (N, K) == (256, 384) and dtype == torch.float32:
        gg = golden("fp8_block")                       # the reference recipe's own output
        wq, ws = I_.quantize_fp8(torch.from_numpy(gg["w"]).to(DEV), L.SCALE_BLOCK128)
        assert torch.equal(ws.cpu(), torch.from_numpy(gg["ws"]))
        assert torch.equal(wq.cpu().view(torch.uint8), torch.from_numpy(gg["wq"]))


def test_cpp_and_python_dispatch_agree(e):
    """The dense linears reach the C ABI through the C++ registration (torch.ops) and, inside the package, through the
    Python host functions (_impl): same checks, same launches, bit-identical results; a shape error is a RuntimeError
    on both routes."""
    g = torch.Generator().manual_seed(11)
    N, K, M = 384, 512, 5
    q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
    s = (0.01 + torch.rand(N, K // 128, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    w = int4.pack_nmajor_i32(q).to(DEV)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    a, b = torch.empty(M, N, dtype=torch.bfloat16, device=DEV), torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    torch.ops.custom_esimd_kernels_vllm.esimd_gemm_int4_pgrp(x, w, s, a)
    e._impl.linear_int4(x, w, s, b)
    assert torch.equal(a, b)
    torch.ops.custom_esimd_kernels_vllm.esimd_gemm_int4_pgrp(x, w.t(), s, a)            # the transposed alias of the same bytes
    assert torch.equal(a, b)
    wq = torch.randint(0, 120, (N, K), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn).to(DEV)
    sc = (0.5 + torch.rand(N, generator=g)).to(DEV)
    torch.ops.custom_esimd_kernels_vllm.esimd_gemv_fp8_pern(x, wq, sc, a, N, K)
    e._impl.linear_fp8(x, wq, sc, b, e._lib.SCALE_CHANNEL, N, K)
    assert torch.equal(a, b)
    with pytest.raises(RuntimeError):
        torch.ops.custom_esimd_kernels_vllm.esimd_gemv_fp8_pern(x, wq, sc, a, N + 1, K)
    with pytest.raises(RuntimeError):
        torch.ops.custom_esimd_kernels_vllm.esimd_gemm_int4_pgrp(x[:, :256], w, s, a)
