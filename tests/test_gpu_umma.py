"""The tcgen05 (tensor-memory) weight-only GEMM, forced on for every shape so that small and ragged
cases run through it too; parity against the CPU oracle with the 1e-2 gate."""
import pytest
import torch

from gpu_util import DEV, assert_close
from oracle import fp8, int4, moe

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def e(lib_built):
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    import custom_esimd_kernels_vllm as pkg
    pkg.set_force_kernel(2)
    yield pkg
    pkg.set_force_kernel(0)
    assert pkg._lib.device_status() == 0, "a bounded device-side wait expired"


def _int4(N, K, sdt, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
    s = (0.002 + torch.randn(N, K // 128, generator=g).abs() * 0.01)
    s = s * torch.where(torch.rand(N, K // 128, generator=g) < 0.3, -1.0, 1.0)
    return q, s.to(sdt)


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (16, 256, 256), (33, 1000, 384), (64, 512, 2048), (200, 384, 512),
                                   (300, 128, 1024), (7, 2560, 2048), (520, 256, 256)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_int4_nmajor(e, M, N, K, dtype):
    q, s = _int4(N, K, dtype, M + N + K)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(dtype)
    ref = int4.linear(x, q, s)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    e.esimd_gemm_int4_pgrp(x.to(DEV), int4.pack_nmajor_i32(q).to(DEV), s.to(DEV), out)
    assert e.last_kernel() in ("umma_wo", "splitk_finalize")
    assert_close(out, ref, what=f"umma int4 M={M} N={N} K={K}")


def test_int4_scale_dtype_differs_from_activation(e):
    q, s = _int4(256, 512, torch.float32, 5)
    x = torch.randn(40, 512).to(torch.bfloat16)
    out = torch.empty(40, 256, dtype=torch.bfloat16, device=DEV)
    e.esimd_gemm_int4_pgrp(x.to(DEV), int4.pack_nmajor_u8(q).to(DEV), s.to(DEV), out)
    assert_close(out, int4.linear(x, q, s), what="umma int4 fp32 scales")


@pytest.mark.parametrize("marlin", [False, True])
@pytest.mark.parametrize("M,N,K", [(16, 128, 256), (70, 384, 640), (256, 1024, 1024)])
def test_int4_kmajor(e, marlin, M, N, K):
    q, s = _int4(N, K, torch.bfloat16, N + K)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    ref = int4.linear(x, q, s)
    wk, sk = int4.to_kmajor(int4.pack_nmajor_i32(q), s, marlin)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    if not marlin:
        e.esimd_gemm_int4_pgrp(x.to(DEV), wk.to(DEV), sk.to(DEV), out)       # classified K-major from the scale shape
    else:
        L = e._lib
        xd, wd, sd = x.to(DEV), wk.to(DEV), sk.to(DEV)
        with L.on_device(out):
            L.check(L.lib.b2q_linear_int4(xd.data_ptr(), L.BF16, K, wd.data_ptr(), L.W4_KMAJOR_MARLIN,
                                          sd.data_ptr(), L.BF16, 1, N, out.data_ptr(), N, M, N, K, 128, None, 0, None))
        torch.cuda.synchronize()
    assert_close(out, ref, what=f"umma int4 kmajor marlin={marlin}")


def test_int4_s4(e):
    q, s = _int4(256, 256, torch.float16, 8)
    x = torch.randn(20, 256).to(torch.float16)
    L = e._lib
    s4 = int4.u4_to_s4_bytes(int4.pack_nmajor_u8(q)).to(DEV)
    xd, sd = x.to(DEV), s.to(DEV)
    out = torch.empty(20, 256, dtype=torch.float16, device=DEV)
    L.check(L.lib.b2q_linear_int4(xd.data_ptr(), L.F16, 256, s4.data_ptr(), L.W4_NMAJOR_S4, sd.data_ptr(), L.F16, 2, 1,
                                  out.data_ptr(), 256, 20, 256, 256, 128, None, 0, None))
    torch.cuda.synchronize()
    assert_close(out, int4.linear(x, q, s), what="umma s4")


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (8, 1536, 5120), (32, 1000, 1024), (64, 512, 2048), (300, 640, 576)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fp8_channel_tensor(e, M, N, K, dtype):
    g = torch.Generator().manual_seed(M + N)
    w = torch.randn(N, K, generator=g) * 0.02
    x = torch.randn(M, K, generator=g).to(dtype)
    wq, s = fp8.quantize_channel(w)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    e.esimd_gemv_fp8_pern(x.to(DEV), wq.to(DEV), s.to(DEV), out, N, K)
    assert e.last_kernel() in ("umma_wo", "splitk_finalize")
    assert_close(out, fp8.linear_channel(x, wq, s), what="umma fp8 channel")
    wq, st = fp8.quantize_tensor(w)
    e.esimd_gemm_fp8_pert(x.to(DEV), wq.to(DEV), st.to(DEV), out)
    assert_close(out, fp8.linear_tensor(x, wq, st), what="umma fp8 tensor")
    w5 = (w / st).to(torch.float8_e5m2)
    e.esimd_gemm_fp8_pert(x.to(DEV), w5.to(DEV), st.to(DEV), out)
    assert_close(out, fp8.linear_tensor(x, w5, st, e5m2=True), what="umma fp8 e5m2")


@pytest.mark.parametrize("M,N,K", [(4, 256, 256), (64, 1000, 5120), (384, 512, 1024)])
def test_fp8_block_w8a16(e, M, N, K):
    g = torch.Generator().manual_seed(M * 7 + N)
    wq, ws = fp8.quantize_block(torch.randn(N, K, generator=g) * 0.3)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    e.esimd_gemm_fp8_blockscale(a.to(DEV), wq.to(DEV), ws.to(DEV), out, 128, 128)
    assert_close(out, fp8.linear_block_w8a16(a, wq, ws), what="umma fp8 block")


def test_fp8_codes_exact_through_tensor_memory(e):
    raw = torch.arange(256, dtype=torch.uint8).view(256, 1).expand(256, 128).contiguous()
    reference = torch.from_numpy(fp8.e4m3_table()) * 128
    finite = torch.isfinite(reference)
    for dtype in (torch.bfloat16, torch.float16):
        x = torch.ones(1, 128, dtype=dtype, device=DEV)
        out = torch.empty(1, 256, dtype=dtype, device=DEV)
        e.esimd_gemv_fp8_pern(x, raw.to(DEV), torch.ones(256, device=DEV), out, 256, 128)
        assert torch.equal(out[0].float().cpu()[finite], reference.to(dtype).float()[finite])


@pytest.mark.parametrize("rows", [[130, 0, 67, 9], [33, 40, 27, 36], [300, 5, 0, 70]])
def test_grouped_int4_and_fp8(e, rows):
    E, N, K = 4, 256, 256
    g = torch.Generator().manual_seed(sum(rows))
    total = sum(rows)
    off = torch.tensor([0] + list(torch.tensor(rows).cumsum(0)), dtype=torch.int32)
    x = (torch.randn(total, K, generator=g) * 0.2).half()
    q = torch.randint(0, 16, (E, N, K), generator=g, dtype=torch.uint8)
    s = (0.002 + torch.randn(E, N, K // 128, generator=g).abs() * 0.01).half()
    out = e.moe_gemm_int4_nmajor(x.to(DEV), int4.pack_nmajor_i32(q).to(DEV), s.to(DEV), off.to(DEV), 128)
    assert e.last_kernel() in ("umma_wo", "splitk_finalize")
    assert_close(out, moe.grouped_linear(x, int4.dequant(q, s, torch.float16), off), what="umma grouped int4")
    wq, ws = fp8.quantize_block(torch.randn(E, N, K, generator=g) * 0.15)
    o8 = torch.empty(total, N, dtype=torch.float16, device=DEV)
    e.esimd_moe_gemm_fp8_blockscale(x.to(DEV), wq.to(DEV), ws.to(DEV), o8, off.to(DEV), N, K, E)
    assert_close(o8, moe.grouped_linear(x, fp8.dequant_block(wq, ws), off), what="umma grouped fp8 block")


def test_moe_prefill_ops_with_ipex_kmajor_marlin_weights(e):
    """The layout moe_prefill_full_int4 takes in the reference: int32 [E, K/8, N], marlin-shuffled."""
    from oracle import configs
    c = configs.c4(seed=3, T=300, E=8, top_k=2, H=256, I=128)
    d13 = int4.dequant(c["q13"], c["s13"], torch.bfloat16)
    d2 = int4.dequant(c["q2"], c["s2"], torch.bfloat16)
    ref = moe.forward(c["x"], c["logits"], d13, d2, 2)
    w13, s13 = int4.to_kmajor(int4.pack_nmajor_i32(c["q13"]), c["s13"], marlin=True)
    w2, s2 = int4.to_kmajor(int4.pack_nmajor_i32(c["q2"]), c["s2"], marlin=True)
    out = e.moe_prefill_full_int4(c["x"].to(DEV), c["logits"].to(DEV), w13.to(DEV), s13.to(DEV), w2.to(DEV), s2.to(DEV), 2, 8)
    # three 16-bit roundings sit between the stages, hence the wider gate for the whole pipeline
    assert_close(out, ref.float(), tol=1e-2, what="moe kmajor marlin")


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 384, 512), (1000, 1000, 1024), (64, 256, 5120)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fp8_block_w8a8(e, M, N, K, dtype):
    """e4m3 x e4m3 tensor cores with per-128-block fp32 promotion, against dq(Aq, As) @ dq(Wq, Ws).T."""
    g = torch.Generator().manual_seed(M + N + K)
    wq, ws = fp8.quantize_block(torch.randn(N, K, generator=g) * 0.02)
    x = torch.randn(M, K, generator=g).to(dtype)
    xq, xs = e.act_quant_fp8_1x128(x.to(DEV))
    rq, rs = fp8.quantize_act_1x128(x)
    assert torch.equal(xq.cpu().view(torch.uint8), rq.view(torch.uint8)) and torch.equal(xs.cpu(), rs)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    e.gemm_fp8_block_w8a8(xq, xs, wq.to(DEV), ws.to(DEV), out)
    assert e.last_kernel() == "umma_w8a8"
    assert_close(out, fp8.linear_block_w8a8(rq, rs, wq, ws), what=f"w8a8 M={M} N={N} K={K}")


@pytest.mark.parametrize("M", [8, 96])
def test_kernel_overlap_modes_give_identical_results(e, M):
    """A chain of dependent linears (each reads what the one before wrote, through the same scratch) must give
    bit-identical results whether consecutive kernels overlap (modes 1, 2) or not (mode 0): strips cut between
    CTAs are summed in a fixed order, so decode shapes are reproducible too."""
    N = K = 4736                                  # 37 strips x 128: ragged last wave, never split at M = 96
    g = torch.Generator().manual_seed(11)
    layers = []
    for i in range(4):
        q, s = _int4(N, K, torch.bfloat16, 100 + i)
        layers.append((int4.pack_nmajor_i32(q).to(DEV), (s * 0.05).to(DEV)))
    wq8 = (torch.randn(N, K, generator=g) * 0.02)
    s8 = (wq8.abs().amax(dim=1) / 448.0).float()
    w8 = (wq8 / s8[:, None]).to(torch.float8_e4m3fn).to(DEV)
    s8 = s8.to(DEV)
    x0 = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    bufs = [torch.empty(M, N, dtype=torch.bfloat16, device=DEV) for _ in range(2)]

    def chain():
        cur = x0
        for w, s in layers:
            e.esimd_gemm_int4_pgrp(cur, w, s, bufs[0])          # never in place: input and output differ
            e.esimd_gemv_fp8_pern(bufs[0], w8, s8, bufs[1], N, K)
            cur = bufs[1]
        return cur.clone()

    results = {}
    try:
        for mode in (0, 1, 2, 0, 2, 1):
            e.set_overlap_mode(mode)
            for _ in range(3):
                r = chain()
            results.setdefault(mode, []).append(r)
    finally:
        e.set_overlap_mode(1)
    torch.cuda.synchronize()
    base = results[0][0].float()
    assert torch.isfinite(base).all()
    for mode, rs in results.items():
        for r in rs:
            assert torch.equal(r, results[0][0]), f"overlap mode {mode} changed the result"


@pytest.mark.parametrize("M,N,K", [(1, 384, 256), (8, 1000, 2048), (13, 4224, 1024), (16, 20000, 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_int4_decode_on_the_int8_mma(e, M, N, K, dtype):
    """The opt-in INT4 decode kernel (unsigned-byte weights x three int8 activation terms, one s32 accumulator per
    group, fp32 promotion): strips cut along k (small N), strips lower than 128 rows, both activation types, and
    the two's-complement nibble layout."""
    q, s = _int4(N, K, dtype, 7 * M + N)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(dtype)
    x[:, 3] *= 300.0
    ref = int4.linear(x, q, s)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    e.set_force_kernel(5)
    try:
        e.esimd_gemm_int4_pgrp(x.to(DEV), int4.pack_nmajor_i32(q).to(DEV), s.to(DEV), out)
        assert e.last_kernel() == "umma_w4_i8"
        assert_close(out, ref, what=f"int8-MMA int4 M={M} N={N} K={K}")
    finally:
        e.set_force_kernel(2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 512, 1024), (1000, 1024, 1024), (64, 256, 5120)])
def test_fp8_block_w8a8_cta_pair_kernel(e, M, N, K):
    """The opt-in CTA-pair variant of the W8A8 GEMM (cluster of two, tcgen05 cta_group::2: one MMA over 256 weight
    rows, each CTA loading its own rows and half of the token tile) against the same oracle as the default kernel."""
    g = torch.Generator().manual_seed(M + N + K)
    w = torch.randn(N, K, generator=g) * 0.3
    wq, ws = fp8.quantize_block(w)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    xq, xs = fp8.quantize_act_1x128(x)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    e.set_force_kernel(6)
    try:
        e.gemm_fp8_block_w8a8(xq.to(DEV), xs.to(DEV), wq.to(DEV), ws.to(DEV), out)
        assert e.last_kernel() == "umma_w8a8_pair"
        assert_close(out, fp8.linear_block_w8a8(xq, xs, wq, ws), what=f"w8a8 pair M={M} N={N} K={K}")
    finally:
        e.set_force_kernel(2)


def test_bounded_wait_gives_up_and_reports(e):
    """Failure detection without a fault: a device-side wait on a barrier nobody arrives on runs out after its limit
    (about a millisecond in this self-test), the kernel records its code in the status word the host reads, returns,
    and the context is still usable for the next launch."""
    L = e._lib
    assert L.device_status() == 0
    # a decode launch whose strips are cut along K (few strips, many SMs): it relies on the arrival counters that the
    # reset below clears together with the status words of every kernel family
    qb, sb = _int4(2048, 4096, torch.bfloat16, 5)
    xb = torch.randn(40, 4096, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(DEV)
    wb, sbd = int4.pack_nmajor_u8(qb).to(DEV), sb.to(DEV)
    before = torch.empty(40, 2048, dtype=torch.bfloat16, device=DEV)
    e.esimd_gemm_int4_pgrp(xb, wb, sbd, before)
    assert L.selftest_bounded_wait(code=777) is True
    assert L.device_status() == 777
    L.device_status_reset()
    assert L.device_status() == 0
    after = torch.empty_like(before)
    e.esimd_gemm_int4_pgrp(xb, wb, sbd, after)
    assert torch.equal(before, after), "a cut-strip launch after the reset differs from the one before it"
    assert_close(after, int4.linear(xb.cpu(), qb, sb), what="cut-strip launch after the reset")
    q, s = _int4(256, 512, torch.bfloat16, 3)
    x = torch.randn(40, 512).to(torch.bfloat16)
    out = torch.empty(40, 256, dtype=torch.bfloat16, device=DEV)
    e.esimd_gemm_int4_pgrp(x.to(DEV), int4.pack_nmajor_u8(q).to(DEV), s.to(DEV), out)
    assert_close(out, int4.linear(x, q, s), what="launch after an expired wait")
    assert L.device_status() == 0
