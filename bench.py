"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--no-configs] [--case NAME]

Headline workload (config.workload = "c2_fp8_channel_gemv_sweep"): the FP8 e4m3 per-output-channel
decode GEMV sweep, weights [27648, 5120], bf16 activations with M in {1, 8, 32}.  One step = one GEMV
at each M, each over a different resident copy of the weight so that no launch finds its weights in
L2 (3 copies x 141.6 MB > 126 MB L2).  metric = weight-streaming GB/s = algorithmic bytes per step
(N*K + 4*N + 2*M*K + 2*M*N per launch) / time.  With N > 1 GPUs every rank owns its own
[27648, 5120] column-parallel shard (no collective on this path): weak scaling, value = sum over ranks.

The same JSON line carries, beside the headline:
  "configs"  (one GPU) the other benchmark configurations, each timed on the device and checked against the CPU oracle
             on a seeded slice of its output first (bench_extra.py): INT4 linear M=16 (C1), FP8 block GEMM as W8A8 and
             w8a16 (C3), the INT4 MoE pipeline (C4), the Llama-70B-shape INT4 decoder layer at M=64 and M=2048 (C5);
             value, unit, roofline_frac, max_rel_err, median and p10/p90.  `--no-configs` leaves the block out.
  "sharded"  (N > 1 GPUs) the forms of the path that need an exchange step (bench_parallel.py): the tensor-parallel
             decoder layer at M=64 and M=2048 (all-reduce after o_proj and down) and the expert-parallel MoE pipeline
             (all-to-all dispatch and combine), with the time spent in the exchange broken out and the one-GPU figure
             of the same case measured in the same run.
  "cpu_baselines"  the reference's CPU torch path (the oracle port) timed per configuration on a bounded sample.

`--impl reference` times the reference's CPU path (torch dequantise-then-matmul, the oracle port) on
the host cores for the same metric on a bounded sample of the same workload.
`--case NAME` runs one of bench_extra's configurations alone and prints its figures (the command the kernel
profiles of that configuration are captured with).
Synthetic seeded data throughout; nothing here reads a dataset or a checkpoint.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "llm-scaler_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

N_W, K_W = 27648, 5120
M_SWEEP = (1, 8, 32)
N_COPIES = 3
METRIC = "fp8_per_channel_gemv_weight_GBps"
# dram__bytes_read.sum + dram__bytes_write.sum of the GEMV kernel, mean of three captured launches of this very
# command under `ncu --set full` (141.8-142.0 MB read, 3.8-4.2 MB written; the writes include L2 write-back of
# what earlier launches left dirty): 1.02 x the algorithmic bytes, i.e. the weights are read exactly once.
NCU_DRAM_BYTES_PER_LAUNCH = 145.85e6


def algo_bytes(M, N=N_W, K=K_W):
    return N * K + 4 * N + 2 * M * K + 2 * M * N


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.stop = index, [], threading.Event()
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [s.strip() for s in out.strip().split(",")]
                if len(parts) >= 7:
                    self.rows.append(parts)
            except Exception:
                pass
            self.stop.wait(0.1)

    def __enter__(self):
        self.t.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.t.join(timeout=6)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(self.rows[0][1]),
                "power_w_max": max(float(r[2]) for r in self.rows), "reasons": reasons, "samples": len(self.rows)}


def dist_setup(n):
    if n <= 1:
        return 0, 1
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    return rank, world


def make_workload(dev, seed):
    """Weights quantised on the GPU with the recipe of the oracle (amax/448 per row), generated per copy."""
    g = torch.Generator(device=dev).manual_seed(seed)
    copies = []
    for _ in range(N_COPIES):
        w = (torch.randn(N_W, K_W, generator=g, device=dev) * 0.02).to(torch.bfloat16).float()
        s = (w.abs().amax(dim=1).clamp(min=1e-12) / 448.0).to(torch.float32)
        copies.append(((w / s[:, None]).to(torch.float8_e4m3fn).contiguous(), s.contiguous()))
        del w
    xs = {M: torch.randn(M, K_W, generator=g, device=dev).to(torch.bfloat16) for M in M_SWEEP}
    outs = {M: torch.empty(M, N_W, dtype=torch.bfloat16, device=dev) for M in M_SWEEP}
    return copies, xs, outs


def run_b200(args):
    import custom_esimd_kernels_vllm as e
    rank, world = dist_setup(args.gpus)
    dev = torch.device("cuda", torch.cuda.current_device())
    assert e._lib.lib.b2q_device_ok() == 0, "this build targets sm_100a (B200) only"
    fp8_peak = None
    if world == 1 and not args.no_configs:
        import bench_extra
        fp8_peak = bench_extra.measure_fp8_peak(dev)     # before anything else heats the package up
    copies, xs, outs = make_workload(dev, 1234 + rank)
    torch.cuda.synchronize()
    # decode serving: the weights are written once (above) and never again, which is what overlap mode 2 asks the
    # caller to promise; a GEMV may then stream its weights while the launch before it is still draining
    e.set_overlap_mode(2)
    op = torch.ops.custom_esimd_kernels_vllm.esimd_gemv_fp8_pern

    def step(i):
        for j, M in enumerate(M_SWEEP):
            wq, s = copies[(i * len(M_SWEEP) + j) % N_COPIES]
            op(xs[M], wq, s, outs[M], N_W, K_W)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # The device-resident loop is what a decode engine runs: the K steps are captured once into a CUDA graph
    # through the same public op (so no host dispatch sits between the launches) and replayed as one unit.
    def capture(nsteps, first):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(nsteps):
                step(first + i)
        return g

    # clocks / throttle reasons are sampled from here to the end of the end-to-end loop: the timed region
    # itself lasts a few milliseconds, too short for nvidia-smi, and everything in this window is the same load
    cs = ClockSampler(torch.cuda.current_device())
    cs.__enter__()
    warm = max(args.warmup, 3)
    for i in range(3):
        step(i)                                    # eager first: one-time kernel attribute set-up cannot be captured
    torch.cuda.synchronize()
    # the launches that are about to be timed, checked against the CPU oracle on a seeded slice of their output
    # (one column out of every 96-row strip a CTA owns, all tokens); the oracle is the checker, nothing of it is timed
    check = None
    if rank == 0:
        from oracle import slices
        cols = slices.pick(N_W, 64, 11, every=96)
        worst = 0.0
        for j, M in enumerate(M_SWEEP):
            wq, s = copies[j % N_COPIES]
            op(xs[M], wq, s, outs[M], N_W, K_W)
            worst = max(worst, slices.fp8_channel_linear(xs[M], wq, s, outs[M], cols)["max_rel_err"])
        check = {"max_rel_err": worst, "how": "%d seeded output columns (one per 96-row strip) x all tokens at each M against "
                                              "oracle.fp8.linear_channel" % cols.numel()}
    launches0 = e.launch_count()
    graph = capture(args.steps, warm)
    launches = e.launch_count() - launches0        # kernels recorded in the graph = kernels per replay
    gwarm = capture(warm, 0)
    gwarm.replay()                                 # W warm-up steps
    graph.replay()                                 # and one untimed pass of the timed graph (uploads it to the device)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    graph.replay()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    # further replays of the same K-step graph, each one sample: the spread of the timed figure
    reps_ms = []
    for _ in range(30):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        reps_ms.append(a.elapsed_time(b))
    reps_ms.sort()
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms = float(t.item())
    step_bytes = sum(algo_bytes(M) for M in M_SWEEP)
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9

    # per-M kernel time (graph of back-to-back launches over rotating copies)
    per_m = {}
    for M in M_SWEEP:
        reps = 30
        gm = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gm):
            for i in range(reps):
                wq, s = copies[i % N_COPIES]
                op(xs[M], wq, s, outs[M], N_W, K_W)
        gm.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        gm.replay()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / reps
        per_m[str(M)] = {"us": round(us, 2), "GBps": round(algo_bytes(M) / us / 1e3, 1),
                         "TFLOPs": round(2.0 * M * N_W * K_W / us / 1e6, 2)}
        del gm

    # end to end through the public op with HOST activations / results (weights are resident state)
    # the step's activations sit in ONE pinned host buffer and travel in ONE copy (three small copies cost three PCIe
    # latencies in front of the first kernel); xe[M] are row ranges of the device copy
    hx_all = torch.cat([xs[M].cpu() for M in M_SWEEP]).pin_memory()
    x_all = torch.empty_like(hx_all, device=dev)
    xe, row = {}, 0
    for M in M_SWEEP:
        xe[M] = x_all[row:row + M]
        row += M
    ho = {M: torch.empty(M, N_W, dtype=torch.bfloat16).pin_memory() for M in M_SWEEP}

    # results go back on a second stream so that the PCIe transfer of one GEMV's output runs under the next GEMV
    main_stream, copy_stream = torch.cuda.current_stream(), torch.cuda.Stream()
    done = {M: torch.cuda.Event() for M in M_SWEEP}

    # largest batch first: its output is 80 % of the step's PCIe bytes and then travels under the two GEMVs behind it
    e2e_order = sorted(M_SWEEP, reverse=True)

    def e2e_step(i):
        x_all.copy_(hx_all, non_blocking=True)
        for j, M in enumerate(e2e_order):
            wq, s = copies[(i * len(M_SWEEP) + j) % N_COPIES]
            op(xe[M], wq, s, outs[M], N_W, K_W)
            done[M].record(main_stream)
            copy_stream.wait_event(done[M])
            with torch.cuda.stream(copy_stream):
                ho[M].copy_(outs[M], non_blocking=True)
        copy_stream.synchronize()                   # the caller reads the results on the host every step
        main_stream.synchronize()

    def timed_e2e(step_fn):
        for i in range(3):
            step_fn(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            step_fn(i)
        barrier()
        t = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return world * step_bytes * args.steps / float(t.item()) / 1e9

    e2e_eager = timed_e2e(e2e_step)

    # The same step as a serving engine issues it: H2D copies, the three op calls and the D2H copies of one step
    # captured once into a CUDA graph (pinned host buffers have fixed addresses), then one replay + one stream
    # synchronisation per step.  All copies and kernels still run every step; only the Python dispatch is gone.
    def capture_e2e(i):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            cur = torch.cuda.current_stream()
            x_all.copy_(hx_all, non_blocking=True)
            for j, M in enumerate(e2e_order):
                wq, s = copies[(i * len(M_SWEEP) + j) % N_COPIES]
                op(xe[M], wq, s, outs[M], N_W, K_W)
                copy_stream.wait_stream(cur)                 # a second branch of the graph: the result's PCIe transfer
                with torch.cuda.stream(copy_stream):         # runs under the next GEMV
                    ho[M].copy_(outs[M], non_blocking=True)
            cur.wait_stream(copy_stream)
        return g

    e2e_graph = capture_e2e(0)      # the weight copy an M uses does not depend on the step index

    def e2e_graph_step(i):
        e2e_graph.replay()
        torch.cuda.current_stream().synchronize()   # the caller reads the results on the host every step

    e2e_value = timed_e2e(e2e_graph_step)
    # keep the GPU under the same load for a moment so that the sampler sees it, then stop sampling
    t_end = time.perf_counter() + 1.0
    i = 0
    while time.perf_counter() < t_end:
        step(i)
        i += 1
    torch.cuda.synchronize()
    cs.__exit__(None, None, None)

    peaks, peak_kind = measured_peaks()
    achieved = step_bytes * args.steps / (ms * 1e-3) / 1e9      # this rank's kernels only
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations x e4m3 weights, fp32 accumulate",
        "data": "synthetic (seeded randn weights ~N(0,0.02) quantised per row, activations ~N(0,1))",
        "config": {"workload": "c2_fp8_channel_gemv_sweep", "N": N_W, "K": K_W, "M_sweep": list(M_SWEEP),
                   "l2": "3 rotating weight copies (425 MB) > 126 MB L2", "sharding": "column-parallel shard per rank, no collective",
                   "overlap_mode": 2,
                   "launch": "K steps captured in one CUDA graph through the public op, one replay timed"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                     "traffic_unit": "DRAM bytes read+written per GEMV launch (one ncu capture of this command)",
                     "algorithmic_bytes_per_launch": round(step_bytes / len(M_SWEEP)), "peak_source": peak_kind,
                     "kernel": e.last_kernel(), "per_M": per_m},
        "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "eager_python_value": round(e2e_eager, 1),
                "how": "per step: one H2D copy of the three activation blocks, the three op calls (largest batch first), D2H of each output on a second stream under the next call, one stream sync; value = the step "
                       "captured as a CUDA graph and replayed, eager_python_value = the same calls issued from Python",
                "h2d_bytes_per_step": sum(2 * M * K_W for M in M_SWEEP),
                "d2h_bytes_per_step": sum(2 * M * N_W for M in M_SWEEP)},
        "gpu_launches": int(launches), "clocks": cs.summary(),
        "max_rel_err": check["max_rel_err"] if check else None, "check": check,
        "replays": {"ms_per_step_median": round(reps_ms[len(reps_ms) // 2] / args.steps, 4),
                    "ms_per_step_p10": round(reps_ms[len(reps_ms) // 10] / args.steps, 4),
                    "ms_per_step_p90": round(reps_ms[(len(reps_ms) * 9) // 10] / args.steps, 4), "samples": len(reps_ms),
                    "how": "30 further replays of the timed K-step graph, this rank"},
    }
    if world == 1 and not args.no_configs:
        import bench_extra
        pk = dict(bench_extra.peaks(), **fp8_peak)
        line["measured_fp8_peak"] = fp8_peak
        line["configs"] = bench_extra.run(e, dev, names=bench_extra.DEFAULT, pk=pk)
    if world > 1:
        import bench_parallel
        line["sharded"] = bench_parallel.run_cases(rank, world, dev)
    if rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline(budget_s=10.0)
        if not args.no_configs:
            line["cpu_baselines"] = cpu_baselines_per_config()
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


def cpu_baseline(budget_s=12.0, threads=None):
    """The reference's CPU path for this workload: dequantise (decode e4m3 * per-row scale) then fp32 matmul,
    on a bounded row-slice of the [27648, 5120] weight, at M = 8; reported in the metric's unit."""
    from oracle import fp8
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    rows = 2048
    w = (torch.randn(rows, K_W, generator=g) * 0.02).to(torch.bfloat16)
    wq, s = fp8.quantize_channel(w)
    x = torch.randn(8, K_W, generator=g).to(torch.bfloat16)
    fp8.linear_channel(x, wq, s)      # warm-up
    n, t0 = 0, time.perf_counter()
    while True:
        fp8.linear_channel(x, wq, s)
        n += 1
        el = time.perf_counter() - t0
        if el > budget_s or n >= 200:
            break
    gbps = n * algo_bytes(8, rows, K_W) / el / 1e9
    # the matmul alone on weights dequantised beforehand (what the CPU path costs once dequantisation is amortised)
    wd = fp8.decode(wq).float() * s[:, None]
    xf = x.float()
    xf @ wd.t()
    m, t1 = 0, time.perf_counter()
    while True:
        xf @ wd.t()
        m += 1
        el2 = time.perf_counter() - t1
        if el2 > budget_s / 4 or m >= 200:
            break
    return {"value": round(gbps, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "matmul_only_value": round(m * algo_bytes(8, rows, K_W) / el2 / 1e9, 3),
            "sample": "%d passes of dequant+matmul over a %d-row slice of the [27648,5120] weight at M=8" % (n, rows)}


def _timed_cpu(fn, budget_s, max_iters=3):
    fn()                                   # warm-up (allocations, thread pool)
    ts = []
    t_all = time.perf_counter()
    while len(ts) < max_iters and (not ts or time.perf_counter() - t_all < budget_s):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return statistics.median(ts), len(ts)


def cpu_baselines_per_config(budget_s=6.0):
    """The reference's CPU torch path (dequantise, then fp32 matmul: the oracle port) for the other configurations, in
    each configuration's own unit, on all host threads.  Every sample is bounded: full width in N and K, a slice of the
    rows (tokens / output rows / experts) sized to a few seconds, stated in `sample`; the figure is throughput, so it
    does not depend on the slice length beyond cache effects."""
    from oracle import configs, fp8, int4, moe
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    out = {"cores": threads, "kind": "port", "what": "dequantise + fp32 matmul per call (the reference's torch path), median of up to 3 calls"}
    c = configs.c1(seed=0)
    t, n = _timed_cpu(lambda: int4.linear(c["x"], c["q"], c["scale"]), budget_s)
    byts = 4096 * 4096 // 2 + 4096 * 32 * 2 + 2 * 16 * 4096 * 2
    out["c1_int4_m16_4096"] = {"value": round(byts / t / 1e9, 3), "unit": "GB/s", "sample": "full size, %d calls" % n}
    c = configs.c3(seed=0, M=512, N=2048)
    xq, xs = fp8.quantize_act_1x128(c["x"])
    t, n = _timed_cpu(lambda: fp8.linear_block_w8a8(xq, xs, c["wq"], c["ws"]), budget_s)
    out["c3_fp8_block_w8a8_m4096"] = {"value": round(2.0 * 512 * 2048 * 5120 / t / 1e12, 4), "unit": "TFLOP/s",
                                      "sample": "512 tokens x 2048 output rows x K=5120 of the [4096 x 17408 x 5120] problem, %d calls" % n}
    t, n = _timed_cpu(lambda: fp8.linear_block_w8a16(c["x"], c["wq"], c["ws"]), budget_s)
    out["c3_fp8_block_w8a16_m4096"] = {"value": round(2.0 * 512 * 2048 * 5120 / t / 1e12, 4), "unit": "TFLOP/s",
                                       "sample": "same slice, activation kept in 16 bit, %d calls" % n}
    c = configs.c4(seed=0, T=512, E=16)
    def moe_call():
        return moe.forward(c["x"], c["logits"], int4.dequant(c["q13"], c["s13"], torch.bfloat16),
                           int4.dequant(c["q2"], c["s2"], torch.bfloat16), 8)
    t, n = _timed_cpu(moe_call, budget_s)
    fl = 512 * 8 * (2.0 * 2048 * 1536 + 2.0 * 768 * 2048)
    out["c4_moe_int4_t4096"] = {"value": round(fl / t / 1e12, 4), "unit": "TFLOP/s", "tokens_per_s": round(512 / t, 1),
                                "sample": "512 tokens over 16 of the 128 experts (top-8, H=2048, I=768), dequantisation included, %d calls" % n}
    for M in (64, 2048):
        g = torch.Generator().manual_seed(M)
        q, s = configs.int4_weight(2048, 8192, g)
        x = torch.randn(min(M, 256), 8192, generator=g).to(torch.bfloat16)
        t, n = _timed_cpu(lambda: int4.linear(x, q, s), budget_s)
        rows = x.shape[0]
        if M == 64:
            byts = 2048 * 8192 // 2 + 2048 * 64 * 2
            out["c5_m64"] = {"value": round(byts / t / 1e9, 3), "unit": "GB/s",
                             "sample": "one [2048 x 8192] row block of the layer's weights at M=64 (the layer is 52 such blocks), %d calls" % n}
        else:
            out["c5_m2048"] = {"value": round(2.0 * rows * 2048 * 8192 / t / 1e12, 4), "unit": "TFLOP/s",
                               "sample": "%d tokens x one [2048 x 8192] row block, %d calls" % (rows, n)}
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step_budget = max(1.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    for _ in range(min(args.warmup, 2)):
        cpu_baseline(budget_s=per_step_budget / 4)
    vals, t0 = [], time.perf_counter()
    for _ in range(args.steps):
        vals.append(cpu_baseline(budget_s=per_step_budget))
    el = time.perf_counter() - t0
    v = statistics.mean(r["value"] for r in vals)
    base = dict(vals[-1], value=round(v, 3))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(v, 3), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(el / max(1, args.steps) * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 matmul of dequantised e4m3",
        "data": "synthetic", "config": {"workload": "c2_fp8_channel_gemv_sweep", "N": N_W, "K": K_W, "M_sweep": list(M_SWEEP)},
        "cpu_baseline": base, "e2e": {"value": round(v, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-configs", action="store_true", help="headline workload only")
    ap.add_argument("--extra", action="store_true", help="accepted for compatibility; the configs block is on by default")
    ap.add_argument("--case", default=None, help="run one configuration of bench_extra.CASES alone")
    args = ap.parse_args()
    if args.case:
        import bench_extra
        import custom_esimd_kernels_vllm as e
        print(json.dumps({"case": args.case, **bench_extra.run(e, torch.device("cuda", 0), only=args.case)}))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
