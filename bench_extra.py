"""Device-timed, result-checked figures for the benchmark configurations other than the headline one.

    python bench.py                    all cases, in the bench line under "configs" (a reduced iteration count keeps the
                                       default run within minutes)
    python bench.py --case c5_m64      one case alone (small enough to profile), printed as one JSON line

Each case reports the quantity its configuration is judged on: weight GB/s for decode shapes, TFLOP/s for
prefill shapes, tokens/s for the MoE pipeline and the decoder layer, with the measured roofline fraction beside
it.  Before a case is timed, one result of exactly the launch that is timed is compared with the CPU oracle on a
seeded slice of its output (oracle/slices.py; the oracle is the checker here, never the thing measured) and the
error is reported as max_rel_err (max|err| / max|ref|).  Timing: CUDA events on the launching stream, warm-up
first, ITERS samples, median with p10 / p90.  Decode-shaped cases are timed the way a serving engine launches
them: REPS calls captured into one CUDA graph through the public op, every replay one sample.
Synthetic seeded data; weights rotate over copies larger than L2 where one copy would fit in it.
"""
import json
import os
import statistics

import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
ITERS = int(os.environ.get("B2Q_BENCH_ITERS", "30"))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def _stats(us):
    us = sorted(us)
    q = lambda f: us[min(len(us) - 1, int(f * len(us)))]
    return {"us": round(statistics.median(us), 2), "us_p10": round(q(0.1), 2), "us_p90": round(q(0.9), 2), "samples": len(us)}


def time_graph(fn, reps, iters=None):
    """reps calls captured into one CUDA graph through the public op; every replay is one sample of us per call."""
    iters = iters or ITERS
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        g.replay()
        b.record()
    torch.cuda.synchronize()
    return _stats([a.elapsed_time(b) * 1e3 / reps for a, b in ev])


def time_eager(fn, iters=None, warm=3):
    iters = iters or ITERS
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for i, (a, b) in enumerate(ev):
        a.record()
        fn(i)
        b.record()
    torch.cuda.synchronize()
    return _stats([a.elapsed_time(b) * 1e3 for a, b in ev])


def measure_fp8_peak(dev, seconds=4.0):
    """Dense e4m3 x e4m3 GEMM throughput of this GPU measured the way MEASURED_PEAKS.json measures bf16:
    torch._scaled_mm 8192^3, best of 10 (burst) and back to back for `seconds` (sustained)."""
    n = 8192
    a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()          # column-major second operand
    one = torch.ones((), device=dev, dtype=torch.float32)
    f = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    for _ in range(3):
        f()
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        f()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    per = max(1, int(seconds * 1e3 / best))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(per):
        f()
    e1.record()
    torch.cuda.synchronize()
    fl = 2.0 * n ** 3
    return {"fp8_tflops": round(fl / best / 1e9, 1), "fp8_tflops_sustained": round(fl * per / e0.elapsed_time(e1) / 1e9, 1),
            "how": "torch._scaled_mm e4m3 x e4m3 8192^3, bf16 out: best of 10 (burst) and %d back to back (sustained)" % per}


def _int4(N, K, dev, g, copies=1, lead=()):
    ws = [torch.randint(-2 ** 31, 2 ** 31 - 1, (*lead, N, K // 8), generator=g, device=dev, dtype=torch.int32)
          for _ in range(copies)]
    s = (0.002 + torch.randn(*lead, N, K // 128, generator=g, device=dev).abs() * 0.01).to(torch.bfloat16)
    return ws, s


def _oracle():
    from oracle import slices          # the checker: compares one result per case, outside every timed region
    return slices


def case_c1(e, dev, g, pk):
    """C1: INT4 linear M=16, K=N=4096 (8.9 MB per launch: launch-latency dominated)."""
    S = _oracle()
    op4 = torch.ops.custom_esimd_kernels_vllm.esimd_gemm_int4_pgrp
    N = K = 4096
    ws, s = _int4(N, K, dev, g, copies=32)                       # 32 x 8.4 MB > 2 x L2
    x = torch.randn(16, K, generator=g, device=dev).to(torch.bfloat16)
    o = torch.empty(16, N, dtype=torch.bfloat16, device=dev)
    op4(x, ws[5], s, o)
    err = S.int4_linear(x, ws[5], s, o, S.pick(N, 256, 1, every=128))
    eager = time_eager(lambda i: op4(x, ws[i % 32], s, o), warm=5)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(1000):                                        # issued back to back from Python, one sync at the end
        op4(x, ws[i % 32], s, o)
    torch.cuda.synchronize()
    stream_us = (time.perf_counter() - t0) * 1e3
    st = time_graph(lambda i: op4(x, ws[i % 32], s, o), 64)
    byts = N * K // 2 + N * (K // 128) * 2 + 16 * K * 2 + 16 * N * 2
    gbs = byts / st["us"] / 1e3
    return {"workload": "int4 g128 linear, M=16, N=K=4096, 32 rotating weight copies", **st,
            "us_eager": eager["us"],                 # CUDA events round one call issued from Python through torch.ops (C++ registration)
            "us_eager_back_to_back": round(stream_us, 2),      # wall clock over 1000 such calls, one synchronize at the end
            "value": round(gbs, 1), "unit": "GB/s", "bound": "hbm", "roofline_frac": round(gbs / pk["hbm_gbs"], 3),
            "algorithmic_bytes": byts, **err, "kernel": e.last_kernel()}


def _c3_weights(e, dev, g, M, N, K):
    w = (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    wq, wsc = e._impl.quantize_fp8(w, e._lib.SCALE_BLOCK128)
    x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    return wq, wsc, x


def case_c3_w8a16(e, dev, g, pk):
    """C3 with the reference's semantics: 128x128 block-scaled e4m3 weights, activation kept in 16 bit."""
    S = _oracle()
    M, N, K = 4096, 17408, 5120
    wq, wsc, x = _c3_weights(e, dev, g, M, N, K)
    o = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    op = torch.ops.custom_esimd_kernels_vllm.esimd_gemm_fp8_blockscale
    op(x, wq, wsc, o, 128, 128)
    err = S.fp8_block_w8a16(x, wq, wsc, o, S.pick(N, 32, 2, every=1024), S.pick(M, 8, 3, every=512))
    st = time_eager(lambda i: op(x, wq, wsc, o, 128, 128))
    fl = 2.0 * M * N * K
    tf = fl / st["us"] / 1e6
    return {"workload": "fp8 128x128 block w8a16 GEMM, M=4096, N=17408, K=5120", **st, "value": round(tf, 1), "unit": "TFLOP/s",
            "bound": "tensor (bf16 MMA)", "roofline_frac": round(tf / pk["bf16_tflops"], 3), **err, "kernel": e.last_kernel()}


def case_c3_w8a8(e, dev, g, pk):
    """C3 as the configuration states it: activations quantised per token per 128 columns, e4m3 x e4m3 MMA."""
    S = _oracle()
    M, N, K = 4096, 17408, 5120
    wq, wsc, x = _c3_weights(e, dev, g, M, N, K)
    o = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    xq, xsc = e.act_quant_fp8_1x128(x)
    e.gemm_fp8_block_w8a8(xq, xsc, wq, wsc, o)
    err = S.fp8_block_w8a8(xq, xsc, wq, wsc, o, S.pick(N, 32, 2, every=1024), S.pick(M, 8, 3, every=512))
    fl = 2.0 * M * N * K
    st = time_eager(lambda i: e.gemm_fp8_block_w8a8(xq, xsc, wq, wsc, o))
    stq = time_eager(lambda i: e.gemm_fp8_block_w8a8(*e.act_quant_fp8_1x128(x), wq, wsc, o))
    tf = fl / st["us"] / 1e6
    fp8_peak = pk.get("fp8_tflops") or 2 * pk["bf16_tflops"]
    return {"workload": "fp8 128x128 block W8A8 GEMM (1x128 activation scales), M=4096, N=17408, K=5120", **st,
            "value": round(tf, 1), "unit": "TFLOP/s", "us_with_act_quant": stq["us"],
            "TFLOPs_with_act_quant": round(fl / stq["us"] / 1e6, 1), "bound": "tensor (fp8 MMA)",
            "roofline_frac": round(tf / fp8_peak, 3),
            "peak": fp8_peak, "peak_source": "measured here (torch._scaled_mm)" if pk.get("fp8_tflops") else "2 x measured bf16 burst",
            **err, "kernel": e.last_kernel()}


C5_SHAPES = {"qkv": (10240, 8192), "o": (8192, 8192), "gate_up": (57344, 8192), "down": (8192, 28672)}


def _case_c5(e, dev, g, pk, M):
    """C5: one Llama-70B-shape decoder layer of INT4 linears on one GPU (attention replaced by the q slice)."""
    S = _oracle()
    op4 = torch.ops.custom_esimd_kernels_vllm.esimd_gemm_int4_pgrp
    layer = {n: _int4(N_, K_, dev, g, copies=1) for n, (N_, K_) in C5_SHAPES.items()}
    wbytes = sum(N_ * K_ // 2 + N_ * (K_ // 128) * 2 for N_, K_ in C5_SHAPES.values())
    params = sum(N_ * K_ for N_, K_ in C5_SHAPES.values())
    x = torch.randn(M, 8192, generator=g, device=dev).to(torch.bfloat16)
    bufs = {n: torch.empty(M, N_, dtype=torch.bfloat16, device=dev) for n, (N_, _) in C5_SHAPES.items()}
    acts = {}

    def layer_fwd(i):
        op4(x, layer["qkv"][0][0], layer["qkv"][1], bufs["qkv"])
        op4(bufs["qkv"][:, :8192], layer["o"][0][0], layer["o"][1], bufs["o"])
        op4(bufs["o"], layer["gate_up"][0][0], layer["gate_up"][1], bufs["gate_up"])
        acts["a"] = e._impl.silu_mul(bufs["gate_up"])
        op4(acts["a"], layer["down"][0][0], layer["down"][1], bufs["down"])

    # every GEMM of the layer against the oracle, each on the input it actually received
    layer_fwd(0)
    torch.cuda.synchronize()
    toks = torch.arange(M) if M <= 64 else S.pick(M, 8, 5, every=512)
    ins = {"qkv": x, "o": bufs["qkv"][:, :8192], "gate_up": bufs["o"], "down": acts["a"]}
    worst = {"max_rel_err": 0.0, "mean_rel_err": 0.0, "cos": 1.0}
    for n, (N_, _) in C5_SHAPES.items():
        er = S.int4_linear(ins[n].contiguous(), layer[n][0][0], layer[n][1], bufs[n], S.pick(N_, 32, 6, every=1024), toks)
        worst = {"max_rel_err": max(worst["max_rel_err"], er["max_rel_err"]),
                 "mean_rel_err": max(worst["mean_rel_err"], er["mean_rel_err"]), "cos": min(worst["cos"], er["cos"])}
    # 428 MB of weights per pass: no L2 residency
    st = time_graph(layer_fwd, 10) if M <= 64 else time_eager(layer_fwd)
    us = st["us"]
    rec = {"workload": "Llama-70B-shape INT4 decoder layer (qkv, o, gate_up, SiLU*mul, down), M=%d, one GPU" % M, **st,
           "us_per_layer": us, "tokens_per_s_80_layers": round(M / (us * 80) * 1e6, 1), **worst}
    if M <= 64:
        gbs = wbytes / us / 1e3
        rec.update(value=round(gbs, 1), unit="GB/s", bound="hbm", roofline_frac=round(gbs / pk["hbm_gbs"], 3))
    else:
        tfl = 2.0 * M * params / us / 1e6
        rec.update(value=round(tfl, 1), unit="TFLOP/s", bound="tensor (bf16 MMA)", roofline_frac=round(tfl / pk["bf16_tflops"], 3))
    rec["kernel"] = e.last_kernel()
    return rec


def case_c4(e, dev, g, pk):
    """C4: INT4 MoE pipeline, 128 experts, top-8, H=2048, I=768, T=4096."""
    S = _oracle()
    T, E, H, I, k = 4096, 128, 2048, 768, 8
    (w13,), s13 = _int4(2 * I, H, dev, g, lead=(E,))
    (w2,), s2 = _int4(H, I, dev, g, lead=(E,))
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=dev).to(torch.bfloat16)
    before = e.launch_count()
    out = e.moe_prefill_full_int4(x, logits, w13, s13, w2, s2, k, E)
    launches = e.launch_count() - before
    err = S.moe_int4(x, logits, w13, s13, w2, s2, k, out, S.pick(T, 12, 7))
    st = time_eager(lambda i: e.moe_prefill_full_int4(x, logits, w13, s13, w2, s2, k, E))
    fl = T * k * (2.0 * H * 2 * I + 2.0 * I * H)
    tf = fl / st["us"] / 1e6
    return {"workload": "INT4 MoE pipeline, T=4096, E=128, top-8, H=2048, I=768", **st, "value": round(tf, 1), "unit": "TFLOP/s",
            "tokens_per_s": round(T / st["us"] * 1e6, 0), "bound": "tensor (bf16 MMA)",
            "roofline_frac": round(tf / pk["bf16_tflops"], 3), "launches_per_pass": int(launches), **err}


def case_c4_decode(e, dev, g, pk):
    """The decode form of C4's pipeline: moe_forward_full_int4 on 16 tokens (128 experts, top-8, H=2048, I=768) with an
    INT4 shared expert of the same width; N-major experts.  Weight bytes touched: up to 128 of the 128 experts."""
    T, E, H, I, k = 16, 128, 2048, 768, 8
    (w13,), s13 = _int4(2 * I, H, dev, g, lead=(E,))
    (w2,), s2 = _int4(H, I, dev, g, lead=(E,))
    (sgu,), sgu_s = _int4(2 * I, H, dev, g)
    (sdn,), sdn_s = _int4(H, I, dev, g)
    sgu_s, sdn_s = sgu_s.t().contiguous(), sdn_s.t().contiguous()          # [K/128, N], as the reference receives them
    gate_w = (torch.randn(1, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=dev).to(torch.bfloat16)
    fn = lambda i: e.moe_forward_full_int4(x, logits, w13, s13, sgu, sgu_s, w2, s2, sdn, sdn_s, gate_w, k, 1, E, True)
    st = time_graph(fn, 10)
    touched = min(E, T * k) * (3 * I * H // 2) + 3 * I * H // 2
    gbs = touched / st["us"] / 1e3
    return {"workload": "moe_forward_full_int4, 16 tokens, INT4 shared expert", **st, "tokens_per_s": round(T / st["us"] * 1e6, 0),
            "value": round(gbs, 1), "unit": "GB/s", "bound": "hbm", "roofline_frac": round(gbs / pk["hbm_gbs"], 3)}


CASES = {
    "c1_int4_m16_4096": case_c1,
    "c3_fp8_block_w8a16_m4096": case_c3_w8a16,
    "c3_fp8_block_w8a8_m4096": case_c3_w8a8,
    "c5_m1": lambda e, dev, g, pk: _case_c5(e, dev, g, pk, 1),
    "c5_m8": lambda e, dev, g, pk: _case_c5(e, dev, g, pk, 8),
    "c5_m64": lambda e, dev, g, pk: _case_c5(e, dev, g, pk, 64),
    "c5_m2048": lambda e, dev, g, pk: _case_c5(e, dev, g, pk, 2048),
    "c4_moe_int4_t4096": case_c4,
    "c4_moe_decode_t16_shared": case_c4_decode,
}
# the cases the default bench line carries: one per benchmark configuration besides the headline
DEFAULT = ("c1_int4_m16_4096", "c3_fp8_block_w8a8_m4096", "c3_fp8_block_w8a16_m4096", "c4_moe_int4_t4096", "c5_m64", "c5_m2048")


def run(e, dev, only=None, names=None, pk=None):
    pk = pk or peaks()
    out = {}
    for name, fn in CASES.items():
        if only is not None and name != only:
            continue
        if only is None and names is not None and name not in names:
            continue
        g = torch.Generator(device=dev).manual_seed(7)
        # the weights of every case are written once, before the timed calls: the serving contract of overlap mode 2
        # (a GEMM may stream weights while the kernel before it drains); an explicit B2Q_OVERLAP_MODE wins
        e.set_overlap_mode(int(os.environ.get("B2Q_OVERLAP_MODE", "2")))
        try:
            out[name] = fn(e, dev, g, pk)
        finally:
            e.set_overlap_mode(1)
        torch.cuda.empty_cache()
    return out
