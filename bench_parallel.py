"""Multi-GPU figures for the two sharded forms of the path: a tensor-parallel INT4 decoder layer (Llama-70B shapes,
M = 64 and M = 2048) and the expert-parallel INT4 MoE pipeline (128 experts, top-8, H = 2048, I = 768, 4096 tokens).

    python bench_parallel.py                                            one GPU (TP1 / EP1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench_parallel.py [--cases tp_m64,tp_m2048,ep]                  N ranks, one per GPU, NCCL

One process per GPU.  Tensor parallel: QKV and gate_up are split by output rows (no communication), o_proj and down by
K in multiples of the 128-group, each followed by an all-reduce (sum) of the [M, 8192] partial results.  Expert
parallel: experts [r * E / G, (r + 1) * E / G) live on rank r, every rank starts with T / G tokens, rows travel by
all-to-all to their experts' rank and back.  Timing: CUDA events on every rank around the same iterations between
barriers, the maximum over ranks is reported.  Synthetic seeded weights (uniform nibbles, scales 0.002 + |N(0, 0.01)|);
attention is replaced by the rank's q slice of the QKV output, as in the single-GPU layer case.  Rank 0 prints one
JSON line per case.
"""
import argparse
import json
import os
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


def _timed(fn, reps, warm, world):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(reps):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) * 1e3 / reps], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())          # microseconds per iteration, slowest rank


def _timed_graph(fn, reps, world):
    """Decode shapes: reps iterations (their all-reduces included) captured into one CUDA graph, one replay timed,
    as a serving engine's decode loop runs them; no Python dispatch between the launches."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    g.replay()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) * 1e3 / reps], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def tp_case(M, rank, world, dev, P, be):
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    layers = 2 if M > 64 else 3          # distinct weights per layer: 428 MB / world each, nothing stays in L2
    stack = [P.TPLayer(qkv=_int4(QKV_N // world, HID, dev, g), o=_int4(HID, HID // world, dev, g),
                       gate_up=_int4(2 * FFN // world, HID, dev, g), down=_int4(HID, FFN // world, dev, g))
             for _ in range(layers)]
    x = torch.randn(M, HID, generator=torch.Generator(device=dev).manual_seed(7), device=dev).to(torch.bfloat16)

    def step(i):
        h = x
        for layer in stack:
            h = P.tp_layer_forward(h, layer, be)
        return h

    how = "eager calls through the public ops (an all-reduce follows o_proj and down)"
    if M <= 64:
        us = _timed_graph(step, 6, world) / layers
        how = "six passes over the layers captured in one CUDA graph, all-reduces included; one replay timed"
    else:
        us = _timed(step, 4, 3, world) / layers
    params = QKV_N * HID + HID * HID + 2 * FFN * HID + HID * FFN
    rec = {"case": f"tp_c5_m{M}", "n_gpus": world, "parallelism": f"tp{world}", "us_per_layer": round(us, 1),
           "tokens_per_s_80_layers": round(M / (us * 80) * 1e6, 1),
           "all_reduce_bytes_per_layer": 2 * M * HID * 2 if world > 1 else 0,
           "launch": how}
    if M <= 64:
        rec["weight_GBps_all_gpus"] = round((params // 2 + params // 128 * 2) / us / 1e3, 1)
    else:
        rec["TFLOPs_all_gpus"] = round(2.0 * M * params / us / 1e6, 1)
    return rec


def ep_case(rank, world, dev, P, be):
    T, E, H, I, k = 4096, 128, 2048, 768, 8
    g = torch.Generator(device=dev).manual_seed(200 + rank)
    w13, s13 = _int4(2 * I, H, dev, g, lead=(E // world,))
    w2, s2 = _int4(H, I, dev, g, lead=(E // world,))
    x = torch.randn(T // world, H, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(T // world, E, generator=g, device=dev).to(torch.bfloat16)
    us = _timed(lambda i: P.ep_moe_forward(x, logits, w13, s13, w2, s2, k, E, be), 5, 2, world)
    fl = T * k * (2.0 * H * 2 * I + 2.0 * I * H)
    return {"case": "ep_c4_moe_int4_t4096", "n_gpus": world, "parallelism": f"ep{world}", "us": round(us, 1),
            "tokens_per_s": round(T / us * 1e6, 0), "TFLOPs_all_gpus": round(fl / us / 1e6, 1),
            "all_to_all_bytes_per_pass": int(2 * T * k * H * 2 * (world - 1) / world),
            "launch": "eager calls; the row counts of the all-to-all are read on the host (two syncs per pass)"}


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
    import custom_esimd_kernels_vllm as pkg                      # noqa: F401  (loads the library or fails loudly)
    from custom_esimd_kernels_vllm import parallel as P
    be = P.CudaBackend()
    # the weights never change during the run: launches may overlap their predecessors' tails (see b2q_set_overlap_mode)
    pkg.set_overlap_mode(int(os.environ.get("B2Q_OVERLAP_MODE", "2")))
    for c in args.cases.split(","):
        if c == "tp_m64":
            rec = tp_case(64, rank, world, dev, P, be)
        elif c == "tp_m2048":
            rec = tp_case(2048, rank, world, dev, P, be)
        elif c == "ep":
            rec = ep_case(rank, world, dev, P, be)
        else:
            raise SystemExit(f"unknown case {c}")
        if rank == 0:
            print(json.dumps(rec), flush=True)
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
