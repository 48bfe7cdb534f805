"""The CPU oracle against golden vectors produced by the reference's own helper functions
(tests/golden/make_golden.py).  Integer / byte results must be identical; dequantised values
are compared bit for bit."""
import numpy as np
import pytest
import torch

from oracle import fp8, int4, moe


def t(a):
    return torch.from_numpy(np.asarray(a))


def test_ggml_q4_0_quantise_pack_dequant(golden):
    g = golden("int4_ggml")
    q, s = int4.quantize_ggml_q4_0(t(g["w"]))
    assert torch.equal(s, t(g["scale"]))
    assert torch.equal(int4.pack_nmajor_u8(q), t(g["packed"]))
    assert torch.equal(int4.unpack_nmajor_u8(t(g["packed"])), q)
    d = int4.dequant(q, s, torch.float16)
    assert torch.equal(d, t(g["deq"]))
    y = int4.linear(t(g["x"]), q, s)
    assert torch.allclose(y, t(g["y"]), rtol=0, atol=1e-5)


def test_nibble_order_and_negative_scale_kat(golden):
    g = golden("int4_ggml")
    q, s = int4.quantize_ggml_q4_0(t(g["kat_w"]))
    assert float(s[0, 0]) == -0.875
    p = int4.pack_nmajor_u8(q)
    assert torch.equal(p, t(g["kat_packed"]))
    # weights [7, -7, 3, -3]: q = [0, 16->15, ...]; low nibble of byte 0 is k = 0
    assert int(p[0, 0]) & 0xF == int(q[0, 0]) and int(p[0, 0]) >> 4 == int(q[0, 1])
    assert torch.equal(int4.dequant(q, s, torch.float16), t(g["kat_deq"]))


def test_symmetric_quantiser_int32_pack_marlin_ipex(golden):
    g = golden("int4_sym")
    q, s = int4.quantize_symmetric(t(g["w"]))
    assert torch.equal(s, t(g["scales"]))
    w32 = int4.pack_nmajor_i32(q)
    assert torch.equal(w32, t(g["qweight"]))
    assert torch.equal(int4.unpack_nmajor_i32(w32), q)
    assert torch.equal(int4.dequant(q, s, torch.float16), t(g["deq"]))
    assert torch.equal(int4.marlin_shuffle_words(w32), t(g["marlin"]))
    wk, sk = int4.to_kmajor(t(g["qe"]), t(g["se"]), marlin=True)
    assert torch.equal(wk, t(g["ipex_q"])) and torch.equal(sk, t(g["ipex_s"]))
    assert torch.equal(int4.unpack_kmajor(wk, True), int4.unpack_nmajor_i32(t(g["qe"])))


def test_uint8_view_aliases_int32_words(golden):
    g = golden("int4_sym")
    q = int4.unpack_nmajor_i32(t(g["qweight"]))
    assert torch.equal(int4.pack_nmajor_u8(q).view(torch.int32), t(g["qweight"]))


def test_cutlass_u4_s4_repack_lossless(golden):
    g = golden("int4_cutlass")
    q = int4.unpack_nmajor_i32(t(g["qe"]))
    u4 = int4.pack_nmajor_u8(q)
    assert torch.equal(u4, t(g["u4"]))
    s4 = int4.u4_to_s4_bytes(u4)
    assert torch.equal(s4, t(g["s4"]))
    d_u = int4.dequant(q, t(g["se"]), torch.float16)
    d_s = int4.dequant_signed(int4.unpack_s4_bytes(s4), t(g["se"]), torch.float16)
    assert torch.equal(d_u, t(g["d_u4"])) and torch.equal(d_s, t(g["d_s4"]))
    assert (d_u.float() - d_s.float()).abs().max() == 0


def test_e4m3_and_e5m2_tables_match_torch_decode(golden):
    g = golden("fp8_block")
    for tab, key in ((fp8.e4m3_table(), "e4m3_codes"), (fp8.e5m2_table(), "e5m2_codes")):
        ref = g[key]
        assert np.array_equal(np.isnan(tab), np.isnan(ref))
        ok = ~np.isnan(ref)
        assert np.array_equal(tab[ok], ref[ok])
        assert np.array_equal(np.signbit(tab[ok]), np.signbit(ref[ok]))
    assert fp8.e4m3_table()[0x80] == 0.0 and np.isnan(fp8.e4m3_table()[0x7F])
    assert np.isfinite(fp8.e4m3_table()).sum() == 254


def test_block_quantiser_and_dequant_with_ragged_edge(golden):
    g = golden("fp8_block")
    wq, ws = fp8.quantize_block(t(g["w"]))
    assert torch.equal(ws, t(g["ws"]))
    assert torch.equal(wq.view(torch.uint8), t(g["wq"]))
    wd = fp8.dequant_block(t(g["wq"]), ws)
    assert torch.equal(wd, t(g["wd"]))
    y = fp8.linear_block_w8a16(t(g["a"]), t(g["wq"]), ws)
    assert torch.allclose(y, t(g["ref"]), rtol=1e-6, atol=1e-6)
    weq, wes = fp8.quantize_block(t(g["we"]))
    assert torch.equal(wes, t(g["wes"])) and torch.equal(weq.view(torch.uint8), t(g["weq"]))
    assert torch.equal(fp8.dequant_block(t(g["weq"]), wes), t(g["wed"]))


def test_block_scale_ownership_for_non_multiple_dims():
    # rows 0..127 belong to block row 0, row 128 to block row 1
    s = torch.tensor([[2.0], [7.0]])
    full = fp8.expand_block_scale(s, 129, 64)
    assert (full[:128] == 2.0).all() and (full[128] == 7.0).all()


def test_moe_forward_matches_reference_per_token_loop(golden):
    g = golden("moe_int4")
    x, logits = t(g["x"]), t(g["logits"])
    d13 = int4.dequant(int4.unpack_nmajor_i32(t(g["q13"])), t(g["s13"]), torch.float16)
    d2 = int4.dequant(int4.unpack_nmajor_i32(t(g["q2"])), t(g["s2"]), torch.float16)
    out = moe.forward(x, logits, d13, d2, int(g["top_k"]), round_intermediates=False)
    ref = t(g["out"]).float()
    err = (out.float() - ref).abs().max() / ref.abs().max()
    assert err < 2e-3, err


def test_moe_decode_pipeline_with_shared_expert_matches_reference_loop(golden):
    """moe_forward_full_int4's reference loop with fp16 and with INT4 shared-expert weights; the packed tensors the
    reference tests hand to the op (K-major marlin experts, column-major repacked shared expert) must unpack to the
    same nibbles."""
    g = golden("moe_int4_shared")
    x, logits, k = t(g["x"]), t(g["logits"]), int(g["top_k"])
    q13, q2 = int4.unpack_nmajor_i32(t(g["q13"])), int4.unpack_nmajor_i32(t(g["q2"]))
    d13 = int4.dequant(q13, t(g["s13"]), torch.float16)
    d2 = int4.dequant(q2, t(g["s2"]), torch.float16)
    out = moe.forward_full(x, logits, d13, d2, t(g["sgu"]), t(g["sdn"]), t(g["sgw"]), k, round_intermediates=False)
    ref = t(g["out_f16"]).float()
    assert (out.float() - ref).abs().max() / ref.abs().max() < 2e-3
    # INT4 shared expert: flat memory of the repacked [K/8, N] tensor is the N-major [N, K/8] matrix
    gq = t(g["sgu_q"]).reshape(t(g["sgu_qn"]).shape)
    dq = t(g["sdn_q"]).reshape(t(g["sdn_qn"]).shape)
    assert torch.equal(gq, t(g["sgu_qn"])) and torch.equal(dq, t(g["sdn_qn"]))
    assert torch.equal(t(g["sgu_s"]).T.contiguous(), t(g["sgu_sn"]))
    sgu_d = int4.dequant(int4.unpack_nmajor_i32(gq), t(g["sgu_sn"]), torch.float16)
    sdn_d = int4.dequant(int4.unpack_nmajor_i32(dq), t(g["sdn_sn"]), torch.float16)
    out = moe.forward_full(x, logits, d13, d2, sgu_d, sdn_d, t(g["sgw"]), k, round_intermediates=False)
    ref = t(g["out_i4"]).float()
    assert (out.float() - ref).abs().max() / ref.abs().max() < 2e-3
    # routed experts: K-major + marlin shuffle unpacks to the same nibbles
    assert torch.equal(int4.unpack_kmajor(t(g["w13_ipex"]), True), q13)
    assert torch.equal(int4.unpack_kmajor(t(g["w2_ipex"]), True), q2)
    assert torch.equal(t(g["s13_ipex"]).permute(0, 2, 1).contiguous(), t(g["s13"]))


def test_route_is_a_stable_counting_sort():
    ids = torch.tensor([[3, 1], [1, 0], [3, 3], [7, 1]], dtype=torch.int32)
    off, tok, p2p, rows = moe.route(ids, 4)   # id 7 is outside [0, 4): dropped
    assert off.tolist() == [0, 1, 4, 4, 7]
    assert tok.tolist() == [3, 1, 2, 7, 0, 4, 5]
    assert p2p.tolist() == [4, 1, 2, 0, 5, 6, -1, 3]
    assert rows.tolist() == [1, 3, 0, 3]


def test_topk_lowest_index_wins_ties():
    logits = torch.zeros(1, 8)
    w, ids = moe.topk_softmax(logits, 3, True, torch.float32)
    assert torch.allclose(w, torch.full((1, 3), 1 / 3))


@pytest.mark.parametrize("M,K", [(1, 128), (4, 256), (16, 128), (256, 512)])
def test_q4_0_device_quantiser_restatement_within_the_reference_envelope(M, K):
    """The reference checks its on-device quantiser against the CPU one through an envelope, not bit for bit
    (tests/test_q4_0_quant_xpu.py:71-121): |scale| within one fp16 ulp, and at most two elements per group whose
    dequantised value differs by more than |scale|.  The restatement of the kernel must sit inside the same envelope
    relative to the tests' Python quantiser, which the golden vectors pin."""
    from oracle import int4
    torch.manual_seed(M * 7 + K)
    x = (torch.randn(M, K) * 0.5).to(torch.bfloat16)
    q_ref, s_ref = int4.quantize_ggml_q4_0(x)
    q_dev, s_dev = int4.quantize_q4_0_device(x)
    ulp = (s_ref.abs().view(torch.int16).to(torch.int32) - s_dev.abs().view(torch.int16).to(torch.int32)).abs()
    assert int(ulp.max()) <= 1
    d_ref = (q_ref.float() - 8) * s_ref.float().repeat_interleave(128, dim=1)
    d_dev = (q_dev.float() - 8) * s_dev.float().repeat_interleave(128, dim=1)
    tol = s_ref.abs().float().repeat_interleave(128, dim=1) + 1e-4
    assert int(((d_ref - d_dev).abs() > tol).sum()) <= 2 * M * (K // 128)
    # and the two agree exactly wherever the fp16 rounding of the scale does not move a rounding boundary
    assert (q_ref == q_dev).float().mean() > 0.99
