"""Generates the golden vectors in this directory by running the REFERENCE's own CPU helper
functions (its tests' pure-PyTorch ground truth), imported from a checkout of intel/llm-scaler.

    python tests/golden/make_golden.py /path/to/llm-scaler

Only this script reads the reference; the committed .npz files are what tests/ load, so the
test-suite itself never needs the checkout.  Every array is small (a few KB).
"""
import importlib
import os
import sys
import types

import numpy as np
import torch

OUT = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    tdir = os.path.join(ref_root, "vllm", "custom-esimd-kernels-vllm", "tests")
    sys.path.insert(0, tdir)
    # the reference tests import the compiled XPU package at module scope; give them an empty stand-in
    sys.modules.setdefault("custom_esimd_kernels_vllm", types.ModuleType("custom_esimd_kernels_vllm"))
    tg = importlib.import_module("test_gemv_int4")
    tm = importlib.import_module("test_moe_int4_kernel")
    tc = importlib.import_module("test_cutlass_nmajor_int4_pack")
    tf = importlib.import_module("test_fp8_blockscale_gemm")
    tp = importlib.import_module("test_fp8_blockscale_moe_prefill")

    # 1. GGML q4_0 quantise / pack / dequant / GEMV  (test_gemv_int4.py:118-233)
    torch.manual_seed(11)
    w = (torch.randn(24, 384) * 0.05).half()
    x = torch.randn(1, 384).half()
    packed, scale = tg.int4_quantize(w)
    deq = tg.int4_dequantize_ref(packed, scale, 24, 384)
    y = tg.gemv_int4_ref(x, packed, scale, 24, 384)
    # nibble-order / scale-sign known-answer case (test_gemv_int4.py:360-414)
    kat_w = torch.zeros(1, 128, dtype=torch.float16)
    kat_w[0, :4] = torch.tensor([7.0, -7.0, 3.0, -3.0], dtype=torch.float16)
    kat_p, kat_s = tg.int4_quantize(kat_w)
    kat_d = tg.int4_dequantize_ref(kat_p, kat_s, 1, 128)
    np.savez_compressed(os.path.join(OUT, "int4_ggml.npz"), w=w.numpy(), x=x.numpy(), packed=packed.numpy(),
             scale=scale.numpy(), deq=deq.numpy(), y=y.numpy(), kat_w=kat_w.numpy(), kat_packed=kat_p.numpy(),
             kat_scale=kat_s.numpy(), kat_deq=kat_d.numpy())

    # 2. symmetric amax/7 quantiser, int32 packing, marlin shuffle, IPEX K-major transform
    #    (test_moe_int4_kernel.py:42-135)
    torch.manual_seed(12)
    w2 = (torch.randn(16, 256) * 0.03).half()
    qw, sc = tm.quantize_int4(w2)
    dq = tm.dequantize_int4(qw, sc, 16, 256)
    shuf = tm.marlin_shuffle_weight(qw.numpy().view(np.uint32))
    E, N, K = 2, 16, 256
    qe = torch.stack([qw, torch.roll(qw, 3, 0)])
    se = torch.stack([sc, torch.roll(sc, 3, 0)])
    qt, st = tm.ipex_transform_expert_weights(qe, se, E, N, K // 8, K // 128)
    np.savez_compressed(os.path.join(OUT, "int4_sym.npz"), w=w2.numpy(), qweight=qw.numpy(), scales=sc.numpy(), deq=dq.numpy(),
             marlin=shuf.view(np.int32), qe=qe.numpy(), se=se.numpy(), ipex_q=qt.numpy(), ipex_s=st.numpy())

    # 3. CUTLASS N-major u4 -> s4 repack (test_cutlass_nmajor_int4_pack.py:26-113)
    u4 = tc._to_cutlass_nmajor(qe)
    s4 = tc._implement_zp_reference(u4)
    d_u4 = tc._decode_cutlass_u4(u4, se, 128)
    d_s4 = tc._decode_cutlass_s4(s4, se, 128)
    np.savez_compressed(os.path.join(OUT, "int4_cutlass.npz"), qe=qe.numpy(), se=se.numpy(), u4=u4.numpy(), s4=s4.numpy(),
             d_u4=d_u4.numpy(), d_s4=d_s4.numpy())

    # 4. FP8 128x128 block quantise / dequant incl. a ragged edge (test_fp8_blockscale_gemm.py:13-36),
    #    all 256 e4m3 codes as torch decodes them (the table test_fp8_blockscale_moe_prefill.py:54-90 checks against),
    #    and the expert-stacked variant (test_fp8_blockscale_moe_prefill.py:18-51)
    torch.manual_seed(13)
    wf = torch.randn(136, 256) * 0.3
    wq, ws = tf.quantize_weight_block(wf)
    wd = tf.dequant_weight(wq, ws)
    a = (torch.randn(5, 256) * 0.5).half()
    ref = a.float() @ wd.t()
    codes = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    codes5 = torch.arange(256, dtype=torch.uint8).view(torch.float8_e5m2).float()
    we = torch.randn(2, 160, 128) * 0.15
    weq, wes = tp.quantize_block(we)
    wed = tp.dequant(weq, wes)
    np.savez_compressed(os.path.join(OUT, "fp8_block.npz"), w=wf.numpy(), wq=wq.view(torch.uint8).numpy(), ws=ws.numpy(),
             wd=wd.numpy(), a=a.numpy(), ref=ref.numpy(), e4m3_codes=codes.numpy(), e5m2_codes=codes5.numpy(),
             we=we.numpy(), weq=weq.view(torch.uint8).numpy(), wes=wes.numpy(), wed=wed.numpy())

    # 5. full MoE forward (test_moe_int4_kernel.py:198-247) with the shared expert zeroed out
    torch.manual_seed(14)
    T, H, I, E, k = 6, 128, 128, 8, 2
    xm = torch.randn(T, H).half()
    logits = torch.randn(T, E).half()
    w13 = (torch.randn(E, 2 * I, H) * 0.05).half()
    w2m = (torch.randn(E, H, I) * 0.05).half()
    q13, s13, q2, s2, d13, d2 = [], [], [], [], [], []
    for e in range(E):
        a_, b_ = tm.quantize_int4(w13[e]); q13.append(a_); s13.append(b_); d13.append(tm.dequantize_int4(a_, b_, 2 * I, H))
        a_, b_ = tm.quantize_int4(w2m[e]); q2.append(a_); s2.append(b_); d2.append(tm.dequantize_int4(a_, b_, H, I))
    d13, d2 = torch.stack(d13), torch.stack(d2)
    out = tm._ref_moe_forward_full(xm, logits, d13, torch.zeros(2 * I, H).half(), d2, torch.zeros(H, I).half(),
                                   torch.zeros(1, H).half(), k, E)
    np.savez_compressed(os.path.join(OUT, "moe_int4.npz"), x=xm.numpy(), logits=logits.numpy(), q13=torch.stack(q13).numpy(),
             s13=torch.stack(s13).numpy(), q2=torch.stack(q2).numpy(), s2=torch.stack(s2).numpy(), out=out.numpy(),
             top_k=np.int32(k))
    # 6. the decode pipeline with the sigmoid-gated shared expert (test_moe_int4_kernel.py:198-247 in full), fp16
    #    and INT4 shared weights, with the packed tensors exactly as the tests hand them to moe_forward_full_int4
    #    (:268-310, :350-420): routed experts K-major + marlin shuffle, INT4 shared expert column-major repacked.
    torch.manual_seed(15)
    T, H, I, IS, E, k = 5, 256, 128, 128, 16, 4
    xs_ = (torch.randn(T, H) * 0.1).half()
    lg = (torch.randn(T, E) * 0.1).half()
    w13 = (torch.randn(E, 2 * I, H) * 0.02).half()
    w2m = (torch.randn(E, H, I) * 0.02).half()
    sgu = (torch.randn(2 * IS, H) * 0.02).half()
    sdn = (torch.randn(H, IS) * 0.02).half()
    sgw = (torch.randn(1, H) * 0.02).half()
    q13, s13, q2, s2, d13, d2 = [], [], [], [], [], []
    for e in range(E):
        a_, b_ = tm.quantize_int4(w13[e]); q13.append(a_); s13.append(b_); d13.append(tm.dequantize_int4(a_, b_, 2 * I, H))
        a_, b_ = tm.quantize_int4(w2m[e]); q2.append(a_); s2.append(b_); d2.append(tm.dequantize_int4(a_, b_, H, I))
    q13, s13, q2, s2 = torch.stack(q13), torch.stack(s13), torch.stack(q2), torch.stack(s2)
    d13, d2 = torch.stack(d13), torch.stack(d2)
    w13_ipex, s13_ipex = tm.ipex_transform_expert_weights(q13, s13, E, 2 * I, H // 8, H // 128)
    w2_ipex, s2_ipex = tm.ipex_transform_expert_weights(q2, s2, E, H, I // 8, I // 128)
    out_f16 = tm._ref_moe_forward_full(xs_, lg, d13, sgu, d2, sdn, sgw, k, E)
    gq, gs = tm.quantize_int4(sgu)
    dq, ds = tm.quantize_int4(sdn)
    out_i4 = tm._ref_moe_forward_full(xs_, lg, d13, tm.dequantize_int4(gq, gs, 2 * IS, H), d2,
                                      tm.dequantize_int4(dq, ds, H, IS), sgw, k, E)
    np.savez_compressed(os.path.join(OUT, "moe_int4_shared.npz"), x=xs_.numpy(), logits=lg.numpy(),
             q13=q13.numpy(), s13=s13.numpy(), q2=q2.numpy(), s2=s2.numpy(),
             w13_ipex=w13_ipex.numpy(), s13_ipex=s13_ipex.numpy(), w2_ipex=w2_ipex.numpy(), s2_ipex=s2_ipex.numpy(),
             sgu=sgu.numpy(), sdn=sdn.numpy(), sgw=sgw.numpy(),
             sgu_q=tm.ipex_column_major_repack(gq.t().contiguous()).numpy(), sgu_s=gs.t().contiguous().numpy(),
             sdn_q=tm.ipex_column_major_repack(dq.t().contiguous()).numpy(), sdn_s=ds.t().contiguous().numpy(),
             sgu_qn=gq.numpy(), sgu_sn=gs.numpy(), sdn_qn=dq.numpy(), sdn_sn=ds.numpy(),
             out_f16=out_f16.numpy(), out_i4=out_i4.numpy(), top_k=np.int32(k))
    print("wrote", sorted(f for f in os.listdir(OUT) if f.endswith(".npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of intel/llm-scaler>")
    main(sys.argv[1])
