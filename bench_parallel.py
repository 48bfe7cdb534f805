"""Multi-GPU figures for the two sharded forms of the path: a tensor-parallel INT4 decoder layer (Llama-70B shapes,
M = 64 and M = 2048) and the expert-parallel INT4 MoE pipeline (128 experts, top-8, H = 2048, I = 768, 4096 tokens).

    python bench_parallel.py                                            one GPU (TP1 / EP1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench_parallel.py [--cases tp_m64,tp_m2048,ep]                  N ranks, one per GPU, NCCL

`bench.py --gpus N` (N > 1) runs the same cases through run_cases() and puts them in its JSON line under "sharded".

One process per GPU.  Tensor parallel: QKV and gate_up are split by output rows (no communication), o_proj and down by
K in multiples of the 128-group, each followed by a sum of the [M, 8192] partial results over the ranks.  Expert
parallel: experts [r * E / G, (r + 1) * E / G) live on rank r, every rank starts with T / G tokens, rows travel by
all-to-all to their experts' rank and back.  Timing: CUDA events on every rank around the same iterations between
barriers, the maximum over ranks is reported.  Beside every sharded figure stand the figure of the same case on ONE GPU
(unsharded weights, measured by rank 0 in the same run) and the time of the exchange step: for tensor parallel the
difference to a run of the same sharded kernels with the sum skipped, for expert parallel CUDA events around the
all-to-alls.  Synthetic seeded weights (uniform nibbles, scales 0.002 + |N(0, 0.01)|); attention is replaced by the
rank's q slice of the QKV output, as in the single-GPU layer case.
"""
import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "llm-scaler_b200"))

HID, QKV_N, FFN = 8192, 10240, 28672


def _int4(N, K, dev, g, lead=()):
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, (*lead, N, K // 8), generator=g, device=dev, dtype=torch.int32)
    s = (0.002 + torch.randn(*lead, N, K // 128, generator=g, device=dev).abs() * 0.01).to(torch.bfloat16)
    return w, s


def _max_over_ranks(v, world):
    t = torch.tensor([v], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _timed(fn, iters, warm, world):
    """Eager calls, one sample per iteration; median over iterations of the slowest rank's time."""
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()          # ranks enter together: the peer-memory exchanges bound their waits (two seconds)
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for i, (a, b) in enumerate(ev):
        a.record()
        fn(i)
        b.record()
    torch.cuda.synchronize()
    us = statistics.median(a.elapsed_time(b) * 1e3 for a, b in ev)
    return _max_over_ranks(us, world)          # microseconds per iteration, slowest rank


def _timed_graph(fn, reps, iters, world):
    """Decode shapes: reps iterations (their exchange steps included) captured into one CUDA graph, every replay one
    sample, as a serving engine's decode loop runs them; no Python dispatch between the launches."""
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()          # ranks enter together: the peer-memory exchanges bound their waits (two seconds)
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i)
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        g.replay()
        b.record()
    torch.cuda.synchronize()
    us = statistics.median(a.elapsed_time(b) * 1e3 / reps for a, b in ev)
    return _max_over_ranks(us, world)


def _tp_stack(world, layers, dev, g, P):
    return [P.TPLayer(qkv=_int4(QKV_N // world, HID, dev, g), o=_int4(HID, HID // world, dev, g),
                      gate_up=_int4(2 * FFN // world, HID, dev, g), down=_int4(HID, FFN // world, dev, g))
            for _ in range(layers)]


def tp_case(M, rank, world, dev, P, be):
    layers = 2 if M > 64 else 3          # distinct weights per layer: 428 MB / world each, nothing stays in L2
    x = torch.randn(M, HID, generator=torch.Generator(device=dev).manual_seed(7), device=dev).to(torch.bfloat16)
    reducer = P.make_reducer(M, HID, torch.bfloat16, dev) if world > 1 else None

    def measure(stack, reduce_fn, w, row_linear=None):
        def step(i):
            h = x
            for layer in stack:
                h = P.tp_layer_forward(h, layer, be, reduce=reduce_fn, row_linear=row_linear)
            return h
        if M <= 64:
            return _timed_graph(step, 4, 10, w) / layers
        return _timed(step, 6, 3, w) / layers

    params = QKV_N * HID + HID * HID + 2 * FFN * HID + HID * FFN
    rec = {"case": f"tp_c5_m{M}", "n_gpus": world, "parallelism": f"tp{world}",
           "launch": "passes over the layers captured in one CUDA graph, exchange steps included; every replay one sample"
                     if M <= 64 else "eager calls through the public ops"}
    # the same case on one GPU: unsharded weights, no exchange (every rank runs it; ranks do not wait for each other here)
    g1 = torch.Generator(device=dev).manual_seed(100)
    one = _tp_stack(1, layers, dev, g1, P)
    us1 = measure(one, lambda t, group=None: t, 1)
    del one
    torch.cuda.empty_cache()
    rec["one_gpu_us_per_layer"] = round(us1, 1)
    if world > 1:
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        stack = _tp_stack(world, layers, dev, g, P)
        us = measure(stack, reducer.reduce, world, getattr(reducer, "row_linear", None))
        us_nosum = measure(stack, lambda t, group=None: t, world)
        if M >= 512:
            ov = P.OverlappedReducer()
            rec["us_per_layer_chunked_all_reduce_under_next_gemm"] = round(measure(stack, ov.reduce, world, ov.row_linear), 1)
            oc = P.OverlappedReducer(chunks=2, split="columns")
            rec["us_per_layer_all_reduce_by_2_column_blocks_under_next_block"] = round(measure(stack, oc.reduce, world, oc.row_linear), 1)
        if isinstance(reducer, P.PeerReducer):
            # for comparison: the same sharded kernels with the process group's all-reduce, and with the two-step form
            # of this library's reduction fed by the GEMM epilogue (the default form for up to four ranks is one step
            # over the links, run behind the GEMM)
            rec["us_per_layer_nccl_all_reduce"] = round(measure(stack, P.NcclReducer().reduce, world), 1)
            two = P.make_reducer(M, HID, torch.bfloat16, dev, kind="peer", mode=2)
            rec["us_per_layer_two_step_fed_by_gemm_epilogue"] = round(measure(stack, two.reduce, world, two.row_linear), 1)
            rec["reduction_status"] = max(reducer.status(), two.status())
            two.close()
        rec.update(us_per_layer=round(us, 1), exchange_us_per_layer=round(max(0.0, us - us_nosum), 1),
                   exchange="sum of the [M, 8192] partial results after o_proj and down: " + reducer.describe(),
                   all_reduce_bytes_per_layer=2 * M * HID * 2, speedup_vs_one_gpu=round(us1 / us, 2),
                   efficiency=round(us1 / us / world, 3))
        if hasattr(reducer, "close"):
            reducer.close()
    else:
        us = us1
        rec["us_per_layer"] = round(us, 1)
    rec["tokens_per_s_80_layers"] = round(M / (us * 80) * 1e6, 1)
    if M <= 64:
        rec["weight_GBps_all_gpus"] = round((params // 2 + params // 128 * 2) / us / 1e3, 1)
    else:
        rec["TFLOPs_all_gpus"] = round(2.0 * M * params / us / 1e6, 1)
    return rec


def ep_case(rank, world, dev, P, be):
    T, E, H, I, k = 4096, 128, 2048, 768, 8
    fl = T * k * (2.0 * H * 2 * I + 2.0 * I * H)

    def build(w, r):
        g = torch.Generator(device=dev).manual_seed(200 + r)
        w13, s13 = _int4(2 * I, H, dev, g, lead=(E // w,))
        w2, s2 = _int4(H, I, dev, g, lead=(E // w,))
        x = torch.randn(T // w, H, generator=g, device=dev).to(torch.bfloat16)
        logits = torch.randn(T // w, E, generator=g, device=dev).to(torch.bfloat16)
        return x, logits, w13, s13, w2, s2

    a1 = build(1, 0)
    import custom_esimd_kernels_vllm as pkg
    us1 = _timed_graph(lambda i: pkg.moe_prefill_full_int4(*a1, k, E), 2, 10, 1)      # the one-GPU pipeline op, as a graph too
    del a1
    torch.cuda.empty_cache()
    rec = {"case": "ep_c4_moe_int4_t4096", "n_gpus": world, "parallelism": f"ep{world}", "one_gpu_us": round(us1, 1)}
    if world > 1:
        a = build(world, rank)
        ex = P.EpExchange(T // world * k, H, torch.bfloat16, dev)
        fwd = lambda marks=None: P.ep_moe_forward_device(*a, k, E, be, ex, marks=marks)
        # nothing in this pass reads a count on the host, so a serving engine can replay it as a CUDA graph
        us = _timed_graph(lambda i: fwd(), 2, 10, world)
        rec["launch"] = "two passes captured in one CUDA graph, exchange included; every replay one sample"
        rec["us_eager"] = round(_timed(lambda i: fwd(), 8, 3, world), 1)
        # for comparison: the same pass with the process group's all-to-all, whose row counts go through the host
        rec["us_nccl_all_to_all_host_counts"] = round(_timed(lambda i: P.ep_moe_forward(*a, k, E, be), 8, 3, world), 1)
        # time inside the exchange steps: events at the phase boundaries of a few further passes
        spans = {"dispatch": [], "combine": []}
        for _ in range(4):
            evs = {}

            def mark(label):
                evs[label] = torch.cuda.Event(enable_timing=True)
                evs[label].record()
            fwd(mark)
            torch.cuda.synchronize()
            spans["dispatch"].append(evs["dispatch_begin"].elapsed_time(evs["dispatch_end"]) * 1e3)
            spans["combine"].append(evs["combine_begin"].elapsed_time(evs["combine_end"]) * 1e3)
        ex_us = _max_over_ranks(statistics.median(spans["dispatch"]) + statistics.median(spans["combine"]), world)
        # the spans include the wait for the slowest rank's rows (ranks drift apart between the synchronised passes)
        rec.update(us=round(us, 1), exchange_us=round(ex_us, 1),
                   exchange="rows and expert indices to the owners (dispatch), results back (combine): " + ex.describe(),
                   exchange_status=ex.status(),
                   all_to_all_bytes_per_pass=int(2 * T * k * H * 2 * (world - 1) / world),
                   speedup_vs_one_gpu=round(us1 / us, 2), efficiency=round(us1 / us / world, 3))
        ex.close()
    else:
        us = us1
        rec["us"] = round(us, 1)
    rec.update(tokens_per_s=round(T / us * 1e6, 0), TFLOPs_all_gpus=round(fl / us / 1e6, 1))
    return rec


def run_cases(rank, world, dev, cases=("tp_m64", "tp_m2048", "ep")):
    """Runs the sharded cases on an initialised process group (or on one GPU) and returns {case name: figures}."""
    import custom_esimd_kernels_vllm as pkg                      # loads the library or fails loudly
    from custom_esimd_kernels_vllm import parallel as P
    be = P.CudaBackend()
    # the weights never change during the run: launches may overlap their predecessors' tails (see b2q_set_overlap_mode)
    pkg.set_overlap_mode(int(os.environ.get("B2Q_OVERLAP_MODE", "2")))
    out = {}
    for c in cases:
        if c == "tp_m64":
            rec = tp_case(64, rank, world, dev, P, be)
        elif c == "tp_m2048":
            rec = tp_case(2048, rank, world, dev, P, be)
        elif c == "ep":
            rec = ep_case(rank, world, dev, P, be)
        else:
            raise SystemExit(f"unknown case {c}")
        out[rec["case"]] = rec
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="tp_m64,tp_m2048,ep")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    res = run_cases(rank, world, dev, tuple(args.cases.split(",")))
    if rank == 0:
        for rec in res.values():
            print(json.dumps(rec), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
