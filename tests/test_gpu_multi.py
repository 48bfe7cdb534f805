"""Tensor-parallel and expert-parallel schedules on two GPUs over NCCL, CUDA kernels underneath, against the
unsharded CPU oracle.  Skipped when fewer than two GPUs are visible."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import configs, int4, moe

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, what, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    try:
        from custom_esimd_kernels_vllm import parallel as P
        be = P.CudaBackend()
        if what in ("tp", "tp_peer", "tp_fused", "tp_overlap"):
            full = configs.c5_layer(seed=3, M=40, tp=1, rank=0, scale=1 / 16)
            packed = {n: (int4.pack_nmajor_i32(full[n][0]), full[n][1]) for n in ("qkv", "o", "gate_up", "down")}
            hidden = full["x"].shape[1]
            qw, qs = packed["qkv"]
            rest = qw.shape[0] - hidden
            rows = torch.cat([torch.arange(rank * hidden // world, (rank + 1) * hidden // world),
                              hidden + torch.arange(rank * rest // world, (rank + 1) * rest // world)])
            to = lambda pair: (pair[0].to(dev), pair[1].to(dev))
            layer = P.TPLayer(qkv=to((qw[rows].contiguous(), qs[rows].contiguous())),
                              o=to(P.shard_row(*packed["o"], rank, world)),
                              gate_up=to(P.shard_column(*packed["gate_up"], rank, world, fused_halves=2)),
                              down=to(P.shard_row(*packed["down"], rank, world)))
            if what == "tp":
                out = P.tp_layer_forward(full["x"].to(dev), layer, be)
            elif what == "tp_overlap":
                # the prefill form: token chunks, the all-reduce of a chunk on a second stream under the next chunk's GEMM
                x = full["x"].to(dev)
                for red in (P.OverlappedReducer(chunks=3, min_chunk_rows=8), P.OverlappedReducer(chunks=2, split="columns")):
                    out = P.tp_layer_forward(x, layer, be, reduce=red.reduce, row_linear=red.row_linear)
            else:
                # the library's own exchange: peer-memory reduction kernel, alone ("tp_peer": the default form for two
                # ranks, one trip over the links) or fed directly by the GEMM epilogue ("tp_fused": the two-step form,
                # the one a GEMM epilogue can feed); three passes so that the flag epochs, both slot sets and both
                # result areas are exercised
                red = P.make_reducer(40, hidden, torch.bfloat16, dev, kind="peer", mode=2 if what == "tp_fused" else 0)
                assert isinstance(red, P.PeerReducer)
                x = full["x"].to(dev)
                for _ in range(3):
                    out = P.tp_layer_forward(x, layer, be, reduce=red.reduce,
                                             row_linear=red.row_linear if what == "tp_fused" else None).clone()
                torch.cuda.synchronize()
                assert red.status() == 0, "a bounded wait of the reduction expired"
                from custom_esimd_kernels_vllm import _lib
                assert _lib.device_status() == 0
                dist.barrier()
                red.close()
        else:
            c = configs.c4(seed=5, T=256, E=8, top_k=2, H=256, I=128)
            T = c["x"].shape[0] // world
            el = 8 // world
            sl, es = slice(rank * T, (rank + 1) * T), slice(rank * el, (rank + 1) * el)
            args = (c["x"][sl].contiguous().to(dev), c["logits"][sl].contiguous().to(dev),
                    int4.pack_nmajor_i32(c["q13"][es]).to(dev), c["s13"][es].contiguous().to(dev),
                    int4.pack_nmajor_i32(c["q2"][es]).to(dev), c["s2"][es].contiguous().to(dev), 2, 8, be)
            if what == "ep":
                out = P.ep_moe_forward(*args)
            else:
                # the library's own exchange over peer memory, counts on the device; three passes on the same buffers
                ex = P.EpExchange(T * 2, c["x"].shape[1], torch.bfloat16, dev)
                for _ in range(3):
                    out = P.ep_moe_forward_device(*args, ex).clone()
                torch.cuda.synchronize()
                assert ex.status() == 0, "a bounded wait of the exchange expired"
                dist.barrier()
                ex.close()
        torch.cuda.synchronize()
        q.put((rank, out.cpu().contiguous().view(torch.int16).numpy().copy()))   # by value: a shared-memory handle dies with the sender
    finally:
        dist.destroy_process_group()


def _run(what):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, what, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        outs = {r: torch.from_numpy(a).view(torch.bfloat16) for r, a in (q.get(timeout=300) for _ in range(world))}
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        # a rank that raised leaves its peer inside an NCCL collective holding a GPU: never leave it running
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
    return outs


@pytest.fixture(scope="module")
def two_gpus(lib_built):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


def _err(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max())


@pytest.mark.timeout(600)
def test_tensor_parallel_layer_two_gpus(two_gpus):
    outs = _run("tp")
    assert torch.equal(outs[0], outs[1])
    full = configs.c5_layer(seed=3, M=40, tp=1, rank=0, scale=1 / 16)
    x = full["x"]
    lin = lambda t, name: int4.linear(t, *full[name]).to(x.dtype)
    h = lin(lin(x, "qkv")[:, :x.shape[1]].contiguous(), "o")
    ref = lin(moe.silu_mul(lin(h, "gate_up")), "down")
    assert _err(outs[0], ref) < 1e-2


@pytest.mark.timeout(600)
@pytest.mark.parametrize("what", ["tp_peer", "tp_fused", "tp_overlap"])
def test_tensor_parallel_layer_two_gpus_own_exchange(two_gpus, what):
    """The same layer with the sum of the row-parallel partial results done by this library's kernels over peer
    memory instead of the process group's all-reduce, or by the chunked all-reduce that overlaps the GEMM; every
    rank must hold bit-identical results."""
    outs = _run(what)
    assert torch.equal(outs[0], outs[1])
    full = configs.c5_layer(seed=3, M=40, tp=1, rank=0, scale=1 / 16)
    x = full["x"]
    lin = lambda t, name: int4.linear(t, *full[name]).to(x.dtype)
    h = lin(lin(x, "qkv")[:, :x.shape[1]].contiguous(), "o")
    ref = lin(moe.silu_mul(lin(h, "gate_up")), "down")
    assert _err(outs[0], ref) < 1e-2


@pytest.mark.timeout(600)
@pytest.mark.parametrize("what", ["ep", "ep_device"])
def test_expert_parallel_two_gpus(two_gpus, what):
    """Experts split over two ranks; rows exchanged by the process group's all-to-all ("ep") or by this library's
    peer-memory kernels with all counts on the device ("ep_device")."""
    outs = _run(what)
    c = configs.c4(seed=5, T=256, E=8, top_k=2, H=256, I=128)
    ref = moe.forward(c["x"], c["logits"], int4.dequant(c["q13"], c["s13"], torch.bfloat16),
                      int4.dequant(c["q2"], c["s2"], torch.bfloat16), 2)
    assert _err(torch.cat([outs[0], outs[1]]), ref) < 1e-2
