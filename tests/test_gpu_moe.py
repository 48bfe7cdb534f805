"""GPU parity of the MoE routing / grouped-GEMM ops against the CPU oracle."""
import pytest
import torch

from gpu_util import DEV, assert_close
from oracle import configs, fp8, int4, moe

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def e(lib_built):
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    import custom_esimd_kernels_vllm as pkg
    return pkg


@pytest.mark.parametrize("T,E,k", [(4096, 128, 8), (33, 256, 8), (7, 128, 10), (5, 64, 2), (1, 8, 8)])
def test_topk(e, T, E, k):
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn(T, E, generator=g).to(torch.float16)
    w, ids = e.moe_topk_softmax(logits.to(DEV), k, E)
    rw, rids = moe.topk_softmax(logits, k, True, torch.float16)
    assert torch.equal(ids.cpu(), rids)
    assert torch.allclose(w.cpu().float(), rw.float(), atol=2e-3, rtol=2e-3)
    tv = torch.empty(T, k, dtype=torch.float16, device=DEV)
    ti = torch.empty(T, k, dtype=torch.int32, device=DEV)
    e.esimd_moe_topk(logits.to(DEV), tv, ti, T)
    assert torch.equal(ti.cpu(), rids)
    w2, i2 = e.moe_topk_int4(logits.to(DEV), k, E, True)
    assert torch.equal(i2.cpu(), rids)


def test_topk_tie_takes_lowest_index(e):
    logits = torch.zeros(3, 128, dtype=torch.float16)
    logits[1, 5] = logits[1, 77] = 2.0
    w, ids = e.moe_topk_softmax(logits.to(DEV), 4, 128)
    assert ids[0].tolist() == [0, 1, 2, 3]
    assert ids[1].tolist() == [5, 77, 0, 1]


@pytest.mark.parametrize("T,E,k", [(4096, 128, 8), (130, 4, 1), (3, 1024, 2), (257, 16, 8)])
def test_route_matches_stable_sort(e, T, E, k):
    g = torch.Generator().manual_seed(T)
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    if E == 4:
        ids[ids == 1] = 0                                   # an empty expert
    off, tok, p2p, rows = e._impl.moe_route(ids.to(DEV), E)
    roff, rtok, rp2p, rrows = moe.route(ids, E)
    assert torch.equal(off.cpu(), roff) and torch.equal(tok.cpu(), rtok)
    assert torch.equal(p2p.cpu(), rp2p) and torch.equal(rows.cpu(), rrows)
    res = torch.ops.moe_int4_prefill_ops.moe_prefill_gather_forward_v2(ids.to(DEV), E)
    assert torch.equal(res[0].cpu(), roff[:E]) and torch.equal(res[1].cpu(), rtok)
    assert torch.equal(res[2].cpu(), rp2p) and torch.equal(res[3].cpu(), rrows)


def test_route_drops_ids_outside_the_local_expert_range(e):
    ids = torch.tensor([[3, 1], [1, 0], [3, 3], [7, 1]], dtype=torch.int32)
    off, tok, p2p, rows = e._impl.moe_route(ids.to(DEV), 4)
    assert off.cpu().tolist() == [0, 1, 4, 4, 7]
    assert tok.cpu().tolist()[:7] == [3, 1, 2, 7, 0, 4, 5]
    assert p2p.cpu().tolist() == [4, 1, 2, 0, 5, 6, -1, 3]


def test_silu_mul_gather_combine(e):
    g = torch.Generator().manual_seed(9)
    gu = torch.randn(77, 256, generator=g).to(torch.bfloat16)
    out = torch.ops.moe_int4_prefill_ops.moe_prefill_silu_mul_forward(gu.to(DEV))
    assert_close(out, moe.silu_mul(gu).float(), tol=4e-3, what="silu_mul")
    x = torch.randn(16, 64, generator=g).to(torch.bfloat16)
    tokens = torch.randperm(64, generator=g).to(torch.int32)
    xp = torch.ops.moe_int4_prefill_ops.moe_prefill_scatter_x_forward(x.to(DEV), tokens.to(DEV), 4)
    assert torch.equal(xp.cpu(), x[(tokens // 4).long()])
    y = torch.randn(64, 128, generator=g).to(torch.bfloat16)
    w = torch.rand(16, 4, generator=g).to(torch.bfloat16)
    o = torch.ops.moe_int4_prefill_ops.moe_prefill_accumulate_forward_v2(y.to(DEV), w.to(DEV))
    assert_close(o, moe.combine(y, w).float(), tol=4e-3, what="accumulate")
    perm = torch.randperm(64, generator=g).to(torch.int32)
    o = torch.ops.moe_int4_prefill_ops.moe_prefill_accumulate_permuted_forward_v2(y.to(DEV), w.to(DEV), perm.to(DEV))
    assert_close(o, moe.combine(y, w, perm).float(), tol=4e-3, what="accumulate permuted")


def _experts_int4(E, N, K, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 16, (E, N, K), generator=g, dtype=torch.uint8)
    s = (0.002 + torch.randn(E, N, K // 128, generator=g).abs() * 0.01).to(dtype)
    return q, s


@pytest.mark.parametrize("rows", [[130, 0, 67, 9], [33, 40, 27, 36], [1, 0, 0, 2], [300, 5, 0, 70]])
def test_grouped_int4_gemm_ragged_and_empty_experts(e, rows):
    E, N, K = 4, 256, 256
    q, s = _experts_int4(E, N, K, torch.float16, sum(rows))
    total = sum(rows)
    off = torch.tensor([0] + list(torch.tensor(rows).cumsum(0)), dtype=torch.int32)
    x = (torch.randn(total, K, generator=torch.Generator().manual_seed(1)) * 0.2).half()
    ref = moe.grouped_linear(x, int4.dequant(q, s, torch.float16), off)
    out = e.moe_gemm_int4_nmajor(x.to(DEV), int4.pack_nmajor_i32(q).to(DEV), s.to(DEV), off.to(DEV), 128)
    assert_close(out, ref, what=f"grouped int4 rows={rows}")
    out = e.moe_gemm_int4_nmajor(x.to(DEV), int4.pack_nmajor_u8(q).to(DEV), s.to(DEV), off.to(DEV), 128)
    assert_close(out, ref, what=f"grouped int4 u8 rows={rows}")


@pytest.mark.parametrize("rows", [[130, 0, 67, 9], [33, 40, 27, 36], [1, 0, 0, 0]])
def test_grouped_fp8_blockscale(e, rows):
    E, N, K = 4, 256, 256
    g = torch.Generator().manual_seed(20260713)
    total = sum(rows)
    off = torch.tensor([0] + list(torch.tensor(rows).cumsum(0)), dtype=torch.int32)
    x = (torch.randn(total, K, generator=g) * 0.2).half()
    wq, ws = fp8.quantize_block(torch.randn(E, N, K, generator=g) * 0.15)
    ref = moe.grouped_linear(x, fp8.dequant_block(wq, ws), off)
    out = torch.empty(total, N, dtype=torch.float16, device=DEV)
    e.esimd_moe_gemm_fp8_blockscale(x.to(DEV), wq.to(DEV), ws.to(DEV), out, off.to(DEV), N, K, E)
    assert_close(out, ref, what=f"grouped fp8 block rows={rows}")


def test_grouped_fp8_e5m2_per_channel_and_per_expert(e):
    E, N, K = 3, 128, 256
    g = torch.Generator().manual_seed(4)
    rows = [17, 0, 50]
    off = torch.tensor([0, 17, 17, 67], dtype=torch.int32)
    x = (torch.randn(67, K, generator=g) * 0.3).half()
    w = torch.randn(E, N, K, generator=g)
    w5 = w.to(torch.float8_e5m2)
    sc = torch.rand(E, N, generator=g) * 0.1 + 0.01
    wd = fp8.decode(w5, e5m2=True) * sc[:, :, None]
    out = torch.empty(67, N, dtype=torch.float16, device=DEV)
    e.esimd_moe_gemm_fp8(x.to(DEV), w5.view(torch.uint8).to(DEV), sc.to(DEV), out, off.to(DEV), N, K, E, 50)
    assert_close(out, moe.grouped_linear(x, wd, off), what="grouped e5m2 per-N")
    st = torch.rand(E, generator=g) * 0.1 + 0.01
    wd = fp8.decode(w5, e5m2=True) * st[:, None, None]
    e.esimd_moe_gemm_fp8_pert(x.to(DEV), w5.view(torch.uint8).to(DEV), st.to(DEV), out, off.to(DEV), N, K, E, 50)
    assert_close(out, moe.grouped_linear(x, wd, off), what="grouped e5m2 per-expert")


def test_scatter_fused_then_gather_roundtrip(e):
    T, K, k, E = 40, 128, 4, 16
    g = torch.Generator().manual_seed(2)
    h = torch.randn(T, K, generator=g).half()
    logits = torch.randn(T, E, generator=g).half()
    tv = torch.empty(T, k, dtype=torch.float16, device=DEV)
    ti = torch.empty(T, k, dtype=torch.int32, device=DEV)
    e.esimd_moe_topk(logits.to(DEV), tv, ti, T)
    sh = torch.empty(T * k, K, dtype=torch.float16, device=DEV)
    sw = torch.empty(T * k, dtype=torch.float16, device=DEV)
    ids = torch.empty(T * k, dtype=torch.int32, device=DEV)
    es = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    mx = torch.empty(1, dtype=torch.int32, device=DEV)
    e.esimd_moe_scatter_fused(h.to(DEV), tv, ti, sh, sw, ids, es, mx, K, k, T, E)
    roff, rtok, rp2p, rrows = moe.route(ti.cpu(), E)
    assert torch.equal(es.cpu(), roff) and int(mx) == int(rrows.max())
    assert torch.equal(sh.cpu(), h[(rtok // k).long()])
    fin = torch.empty(T, K, dtype=torch.float16, device=DEV)
    e.esimd_moe_gather(sh, ids.view(T, k), sw, fin, K, k, T)
    # identity experts: gather of the scattered rows = sum_s w[t, s] * h[t] = h[t] (weights renormalised)
    assert_close(fin, h.float() * tv.cpu().float().sum(1, keepdim=True), tol=4e-3, what="scatter/gather")


def test_moe_pipeline_golden_and_ops(e, golden):
    g = golden("moe_int4")
    x, logits = torch.from_numpy(g["x"]), torch.from_numpy(g["logits"])
    q13, s13 = torch.from_numpy(g["q13"]), torch.from_numpy(g["s13"])
    q2, s2 = torch.from_numpy(g["q2"]), torch.from_numpy(g["s2"])
    k, E = int(g["top_k"]), q13.shape[0]
    out = e.moe_prefill_full_int4(x.to(DEV), logits.to(DEV), q13.to(DEV), s13.to(DEV), q2.to(DEV), s2.to(DEV), k, E)
    # 16-bit roundings between the stages: wider gate for the whole pipeline than for one GEMM
    assert_close(out, torch.from_numpy(g["out"]).float(), tol=1e-2, what="moe golden")


@pytest.mark.parametrize("T", [64, 700])
def test_moe_pipeline_config4_shape_reduced(e, T):
    c = configs.c4(seed=T, T=T, E=16, top_k=4, H=512, I=256)
    d13 = int4.dequant(c["q13"], c["s13"], torch.bfloat16)
    d2 = int4.dequant(c["q2"], c["s2"], torch.bfloat16)
    ref = moe.forward(c["x"], c["logits"], d13, d2, 4)
    out = e.moe_prefill_full_int4(c["x"].to(DEV), c["logits"].to(DEV), int4.pack_nmajor_i32(c["q13"]).to(DEV),
                                  c["s13"].to(DEV), int4.pack_nmajor_i32(c["q2"]).to(DEV), c["s2"].to(DEV), 4, 16)
    assert_close(out, ref.float(), tol=1e-2, what=f"moe T={T}")


@pytest.mark.parametrize("rows_per,E,I,H,dt", [(150, 8, 768, 512, torch.bfloat16), (150, 8, 256, 384, torch.float16),
                                               (5, 16, 128, 256, torch.bfloat16), (40, 4, 640, 256, torch.bfloat16)])
def test_gated_input_grouped_gemm_equals_silu_mul_then_gemm(e, rows_per, E, I, H, dt):
    """The down GEMM fed the un-activated gate_up rows (B2Q_ACT_SILU_MUL_IN) must give, bit for bit, what the separate
    silu_mul op followed by the plain grouped GEMM gives, on the tcgen05 path (many rows per expert) and on the
    few-rows path alike; and both agree with the oracle."""
    I_, L = e._impl, e._lib
    g = torch.Generator().manual_seed(rows_per * 31 + E)
    counts = torch.randint(max(rows_per - 4, 0), rows_per + 5, (E,), generator=g)
    counts[1] = 0
    off = torch.zeros(E + 1, dtype=torch.int32)
    off[1:] = counts.cumsum(0)
    rows = int(off[-1])
    gate_up = (torch.randn(rows, 2 * I, generator=g) * 1.5).to(dt)
    qs = [int4.quantize_symmetric((torch.randn(H, I, generator=g) * 0.05).to(dt)) for _ in range(E)]
    q = torch.stack([a for a, _ in qs])
    s = torch.stack([b for _, b in qs]).to(dt)
    w = torch.stack([int4.pack_nmajor_i32(a) for a in q])
    args = (w.to(DEV), s.to(DEV), off.to(DEV), rows)
    fused = I_.moe_gemm_int4(gate_up.to(DEV), *args, act=L.ACT_SILU_MUL_IN)
    inter = I_.silu_mul(gate_up.to(DEV))
    plain = I_.moe_gemm_int4(inter, *args)
    assert torch.equal(fused, plain)
    ref_inter = moe.silu_mul(gate_up)
    assert torch.allclose(inter.cpu().float(), ref_inter.float(), rtol=1e-2, atol=1e-3)
    ref = torch.empty(rows, H, dtype=dt)
    for x in range(E):
        a, b = int(off[x]), int(off[x + 1])
        if b > a:
            ref[a:b] = int4.linear(ref_inter[a:b], q[x], s[x])
    assert_close(fused, ref, what="gated-input grouped GEMM")
    # a strided source (the gate_up rows living inside a wider buffer) is read through ldx
    wide = torch.zeros(rows, 2 * I + 64, dtype=dt)
    wide[:, :2 * I] = gate_up
    v = wide.to(DEV)[:, :2 * I]
    assert torch.equal(I_.moe_gemm_int4(v, *args, act=L.ACT_SILU_MUL_IN), plain)


def _g(golden, name):
    g = golden(name)
    return {k: torch.from_numpy(g[k]) for k in g.files}


def _rel(a, ref):
    return float((a.float().cpu() - ref.float()).abs().max() / ref.float().abs().max())


def test_decode_pipeline_with_shared_expert_golden(e, golden):
    """moe_forward_full_int4 on the tensors the reference's own tests build (K-major marlin experts; 16-bit or
    column-major repacked INT4 shared expert) against outputs of the reference's per-token loop."""
    g = _g(golden, "moe_int4_shared")
    k, E = int(g["top_k"]), g["q13"].shape[0]
    d = lambda n: g[n].to(DEV)
    empty = torch.empty(0, dtype=torch.float16, device=DEV)
    out = e.moe_forward_full_int4(d("x"), d("logits"), d("w13_ipex"), d("s13_ipex"), d("sgu"), empty,
                                  d("w2_ipex"), d("s2_ipex"), d("sdn"), empty, d("sgw"), k, 1, E, False)
    assert _rel(out, g["out_f16"]) < 1e-2
    out = e.moe_forward_full_int4(d("x"), d("logits"), d("w13_ipex"), d("s13_ipex"), d("sgu_q"), d("sgu_s"),
                                  d("w2_ipex"), d("s2_ipex"), d("sdn_q"), d("sdn_s"), d("sgw"), k, 1, E, False)
    assert _rel(out, g["out_i4"]) < 1e-2
    # N-major (GGML) experts give the same result as the K-major ones
    out_n = e.moe_forward_full_int4(d("x"), d("logits"), d("q13"), d("s13"), d("sgu_q"), d("sgu_s"),
                                    d("q2"), d("s2"), d("sdn_q"), d("sdn_s"), d("sgw"), k, 1, E, True)
    assert _rel(out_n, g["out_i4"]) < 1e-2
    # two's-complement N-major bytes + 16-bit shared expert
    s4 = lambda n: int4.u4_to_s4_bytes(int4.pack_nmajor_u8(int4.unpack_nmajor_i32(g[n]))).to(DEV)
    out_c = e.moe_forward_cutlass_nmajor_int4_full(d("x"), d("logits"), s4("q13"), d("s13"), s4("q2"), d("s2"),
                                                   d("sgu"), d("sdn"), d("sgw"), k, 1, E)
    assert _rel(out_c, g["out_f16"]) < 1e-2
    # no shared expert: the routed part alone
    out_0 = e.moe_forward_full_int4(d("x"), d("logits"), d("w13_ipex"), d("s13_ipex"), empty, empty,
                                    d("w2_ipex"), d("s2_ipex"), empty, empty, empty, k, 0, E, False)
    d13 = int4.dequant(int4.unpack_nmajor_i32(g["q13"]), g["s13"], torch.float16)
    d2 = int4.dequant(int4.unpack_nmajor_i32(g["q2"]), g["s2"], torch.float16)
    assert _rel(out_0, moe.forward(g["x"], g["logits"], d13, d2, k)) < 1e-2


@pytest.mark.parametrize("T,H,E", [(1, 256, 16), (4, 2048, 256), (16, 2048, 16), (3, 3072, 256)])
def test_int4_router_both_layouts(e, T, H, E):
    """moe_router_forward_int4 (tests/test_moe_int4_kernel.py:146-190): weight [E, K/8] directly or shaped [K/8, E]
    over the same memory, scales [K/128, E]; and the GGML presentation with scales [E, K/128].  E == K/128 is the
    case where the two scale layouts have the same shape."""
    gen = torch.Generator().manual_seed(T + H + E)
    w = (torch.randn(E, H, generator=gen) * 0.02).half()
    q, s = int4.quantize_symmetric(w)
    x = (torch.randn(T, H, generator=gen) * 0.1).half()
    ref = int4.linear(x, q, s)
    qw = int4.pack_nmajor_i32(q)
    sc = s.t().contiguous()
    for shaped in (qw, qw.flatten().reshape(H // 8, E)):
        out = e.moe_router_forward_int4(x.to(DEV), shaped.to(DEV), sc.to(DEV), False)
        assert tuple(out.shape) == (T, E)
        assert_close(out, ref, what="router logits")
    out = e.moe_router_forward_int4(x.to(DEV), int4.pack_nmajor_u8(q).to(DEV), s.to(DEV), True)
    assert_close(out, ref, what="router logits, GGML layout")
    wts, ids = e.moe_router_topk_int4(x.to(DEV), qw.to(DEV), sc.to(DEV), False, 4, E, True)
    rw, rids = moe.topk_softmax(out.cpu(), 4, True, torch.float16)
    assert torch.equal(ids.cpu(), rids)
    zero = e.moe_router_forward_int4(torch.zeros(1, H, dtype=torch.float16, device=DEV), qw.to(DEV), sc.to(DEV), False)
    assert float(zero.abs().max()) == 0.0


@pytest.mark.parametrize("T,H,I,dt", [(2, 256, 128, torch.float16), (33, 2048, 256, torch.bfloat16)])
def test_shared_expert_nmajor_signed_nibbles(e, T, H, I, dt):
    gen = torch.Generator().manual_seed(T * H)
    gu = (torch.randn(2 * I, H, generator=gen) * 0.02).to(dt)
    dn = (torch.randn(H, I, generator=gen) * 0.02).to(dt)
    gw = (torch.randn(1, H, generator=gen) * 0.05).to(dt)
    x = (torch.randn(T, H, generator=gen) * 0.5).to(dt)
    (qg, sg), (qd, sd) = int4.quantize_symmetric(gu), int4.quantize_symmetric(dn)
    sg, sd = sg.to(dt), sd.to(dt)
    s4 = lambda q: int4.u4_to_s4_bytes(int4.pack_nmajor_u8(q)).to(DEV)
    out = e.moe_shared_expert_forward_int4_nmajor(x.to(DEV), s4(qg), sg.to(DEV), s4(qd), sd.to(DEV), gw.to(DEV))
    ref = moe.shared_expert(x, int4.dequant(qg, sg, dt), int4.dequant(qd, sd, dt), gw).to(dt)
    assert _rel(out, ref) < 1e-2
    # the gate-add kernel on its own: bit-level check against fp32 arithmetic with one rounding
    y = torch.randn(T, H, generator=gen).to(dt)
    r = torch.randn(T, H, generator=gen).to(dt)
    got = e._impl.moe_shared_gate_add(x.to(DEV), gw.to(DEV), y.to(DEV), r.to(DEV))
    gate = torch.sigmoid(x.float() @ gw.float().T)
    want = (r.float() + gate * y.float()).to(dt)
    assert torch.allclose(got.cpu().float(), want.float(), rtol=1e-2, atol=1e-2)
    assert (got.cpu() != want).float().mean() < 0.02
