"""Tensor-parallel and expert-parallel schedules on two gloo ranks (CPU).  The collectives and the sharding
arithmetic are the product's (custom_esimd_kernels_vllm.parallel); the compute backend is the CPU oracle, so
the test checks that sharded execution reproduces the unsharded oracle."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import configs, int4, moe


class OracleBackend:
    """Same interface as parallel.CudaBackend, computed with the CPU oracle."""

    def linear_int4(self, x, w, s):
        return int4.linear(x, int4.unpack_nmajor_i32(w), s).to(x.dtype)

    def silu_mul(self, g):
        return moe.silu_mul(g)

    def topk(self, logits, k, dtype):
        return moe.topk_softmax(logits, k, True, dtype)

    def route(self, ids, E):
        return moe.route(ids, E)

    def gather_rows(self, src, idx, div):
        return src[(idx // div).long()]

    def expert_mlp(self, x, w13, s13, w2, s2, offsets, tokens, rows):
        d13 = int4.dequant(int4.unpack_nmajor_i32(w13), s13, x.dtype)
        d2 = int4.dequant(int4.unpack_nmajor_i32(w2), s2, x.dtype)
        xs = x[tokens.long()]
        inter = moe.silu_mul(moe.grouped_linear(xs, d13, offsets).to(x.dtype))
        ys = moe.grouped_linear(inter, d2, offsets).to(x.dtype)
        y = torch.zeros(rows, ys.shape[1], dtype=ys.dtype)       # `rows` may be an upper bound (fixed-capacity receive area)
        y[tokens.long()] = ys
        return y

    def combine(self, y, weights, perm, T, k):
        return moe.combine(y, weights, perm)


class HostExchange:
    """Stand-in for parallel.EpExchange on CPU ranks: the same interface and the same buffer layout (a receive area
    of world x cap rows with one slot per source rank, expert index -1 in unused positions, a return area in the
    source's send order), moved by gloo all-to-alls.  It lets the host-side arithmetic of ep_moe_forward_device
    (destination sort, local expert indices, upper-bound row counts, combine from the return area) run against the
    CPU oracle; the peer-memory kernels themselves are tested on GPUs."""

    def __init__(self, cap, H, dtype):
        self.world, self.rank, self.cap = dist.get_world_size(), dist.get_rank(), cap
        self.recv_rows = torch.zeros(self.world * cap, H, dtype=dtype)
        self.recv_ids = torch.full((self.world * cap,), -1, dtype=torch.int32)
        self.ret_rows = torch.zeros(cap, H, dtype=dtype)

    def dispatch(self, x, order, top_k, offsets, local_ids):
        W, cap = self.world, self.cap
        self.sc = (offsets[1:] - offsets[:-1]).tolist()
        sc = torch.tensor(self.sc, dtype=torch.int64)
        rc = torch.empty_like(sc)
        dist.all_to_all_single(rc, sc)
        self.rc = rc.tolist()
        rows = x[(order // top_k).long()].contiguous()
        got = torch.empty(sum(self.rc), x.shape[1], dtype=x.dtype)
        got_e = torch.empty(sum(self.rc), dtype=torch.int32)
        dist.all_to_all_single(got, rows, self.rc, self.sc)
        dist.all_to_all_single(got_e, local_ids.contiguous(), self.rc, self.sc)
        self.recv_ids.fill_(-1)
        at = 0
        for s_ in range(W):
            n = self.rc[s_]
            self.recv_rows[s_ * cap:s_ * cap + n] = got[at:at + n]
            self.recv_ids[s_ * cap:s_ * cap + n] = got_e[at:at + n]
            at += n

    def wait(self, phase, like):
        pass

    def give_back(self, y):
        cap = self.cap
        send = torch.cat([y[s_ * cap:s_ * cap + self.rc[s_]] for s_ in range(self.world)]).contiguous()
        back = torch.empty(sum(self.sc), y.shape[1], dtype=y.dtype)
        dist.all_to_all_single(back, send, self.sc, self.rc)
        self.ret_rows[:back.shape[0]] = back


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, what, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    try:
        from custom_esimd_kernels_vllm import parallel as P
        be = OracleBackend()
        if what == "tp":
            full = configs.c5_layer(seed=3, M=5, tp=1, rank=0, scale=1 / 16)     # hidden 512
            packed = {n: (int4.pack_nmajor_i32(full[n][0]), full[n][1]) for n in ("qkv", "o", "gate_up", "down")}
            # column split of QKV keeps the rank's q slice in front: split q, k, v separately like heads
            hidden = full["x"].shape[1]
            qw, qs = packed["qkv"]
            q_rows = torch.arange(rank * hidden // world, (rank + 1) * hidden // world)
            kv_rows = hidden + torch.arange(rank * (qw.shape[0] - hidden) // world, (rank + 1) * (qw.shape[0] - hidden) // world)
            rows = torch.cat([q_rows, kv_rows])
            layer = P.TPLayer(qkv=(qw[rows].contiguous(), qs[rows].contiguous()),
                              o=P.shard_row(*packed["o"], rank, world),
                              gate_up=P.shard_column(*packed["gate_up"], rank, world, fused_halves=2),
                              down=P.shard_row(*packed["down"], rank, world))
            out = P.tp_layer_forward(full["x"], layer, be)
            q.put((rank, _pack(out)))
        elif what.startswith("guard"):
            # a collective that returns NaN from finite input, as the reference's repair path assumes: rank 1's
            # first `fail` calls (all of them for "guard_fallback") poison the result
            fail = {"guard_once": 1, "guard_fallback": 10 ** 6, "guard_clean": 0}[what]
            calls = {"n": 0}

            def flaky(t, g):
                dist.all_reduce(t, op=dist.ReduceOp.SUM, group=g)
                calls["n"] += 1
                if rank == 1 and calls["n"] <= fail:
                    t[0, 0] = float("nan")
            x = torch.full((4, 8), float(rank + 1)).to(torch.bfloat16)
            stats = {}
            out = P.guarded_all_reduce(x, collective=flaky, stats=stats)
            q.put((rank, _pack(out), stats, calls["n"]))
            return
        else:
            c = configs.c4(seed=5, T=24, E=8, top_k=2, H=128, I=128)
            T = c["x"].shape[0] // world
            e_local = 8 // world
            sl = slice(rank * T, (rank + 1) * T)
            es = slice(rank * e_local, (rank + 1) * e_local)
            args = (c["x"][sl].contiguous(), c["logits"][sl].contiguous(),
                    int4.pack_nmajor_i32(c["q13"][es]), c["s13"][es].contiguous(),
                    int4.pack_nmajor_i32(c["q2"][es]), c["s2"][es].contiguous(), 2, 8, be)
            if what == "ep_device":
                out = P.ep_moe_forward_device(*args, HostExchange(T * 2, c["x"].shape[1], torch.bfloat16))
            else:
                out = P.ep_moe_forward(*args)
            q.put((rank, _pack(out)))
    finally:
        dist.destroy_process_group()


def _pack(t):
    """Results cross the process boundary by value: a tensor in a multiprocessing queue travels as a shared-memory
    handle that dies with the sending process."""
    assert t.dtype == torch.bfloat16
    return t.contiguous().view(torch.int16).numpy().copy()


def _unpack(a):
    return torch.from_numpy(a).view(torch.bfloat16)


def _run(what):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, what, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        outs = {}
        for _ in range(world):
            item = q.get(timeout=120)
            outs[item[0]] = _unpack(item[1]) if len(item) == 2 else (_unpack(item[1]),) + tuple(item[2:])
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        # a rank that raised leaves its peer inside a collective: never leave it running
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
    return outs


@pytest.mark.timeout(300)
def test_tensor_parallel_layer_matches_unsharded(lib_built):
    outs = _run("tp")
    assert torch.equal(outs[0], outs[1])                       # all-reduced result is replicated
    from custom_esimd_kernels_vllm import parallel as P
    full = configs.c5_layer(seed=3, M=5, tp=1, rank=0, scale=1 / 16)
    packed = {n: (int4.pack_nmajor_i32(full[n][0]), full[n][1]) for n in ("qkv", "o", "gate_up", "down")}
    one = P.TPLayer(qkv=packed["qkv"], o=packed["o"], gate_up=packed["gate_up"], down=packed["down"])
    ref = P.tp_layer_forward(full["x"], one, OracleBackend())
    err = (outs[0].float() - ref.float()).abs().max() / ref.float().abs().max()
    assert err < 2e-2, err                                     # two extra 16-bit roundings of the partial sums


@pytest.mark.timeout(300)
@pytest.mark.parametrize("what", ["ep", "ep_device"])
def test_expert_parallel_matches_single_rank(lib_built, what):
    """"ep": the all-to-all form with host counts; "ep_device": the form whose exchange keeps every count on the
    device (fixed-capacity slots, upper-bound row counts), here over a CPU stand-in for the peer-memory kernels."""
    outs = _run(what)
    c = configs.c4(seed=5, T=24, E=8, top_k=2, H=128, I=128)
    ref = moe.forward(c["x"], c["logits"], int4.dequant(c["q13"], c["s13"], torch.bfloat16),
                      int4.dequant(c["q2"], c["s2"], torch.bfloat16), 2)
    got = torch.cat([outs[0], outs[1]])
    assert torch.equal(got, ref)                               # same arithmetic in the same order per token


def test_shard_helpers():
    from custom_esimd_kernels_vllm import parallel as P
    w = torch.arange(16 * 64, dtype=torch.int32).reshape(16, 64)         # N=16, K=512
    s = torch.arange(16 * 4, dtype=torch.float32).reshape(16, 4)
    w0, s0 = P.shard_column(w, s, 1, 2, fused_halves=2)
    assert w0[:, 0].tolist() == [w[r, 0].item() for r in (4, 5, 6, 7, 12, 13, 14, 15)]
    w1, s1 = P.shard_row(w, s, 1, 2)
    assert w1.shape == (16, 32) and s1.shape == (16, 2) and w1[0, 0] == w[0, 32] and s1[0, 0] == s[0, 2]


@pytest.mark.timeout(300)
@pytest.mark.parametrize("what,retries,fallback", [("guard_clean", 0, False), ("guard_once", 1, False), ("guard_fallback", 3, True)])
def test_guarded_all_reduce_repairs_a_nan(lib_built, what, retries, fallback):
    """One rank's collective returns a NaN: every rank learns of it, all repeat the collective, and when the NaN
    persists the all-gather + local sum takes over; both ranks end with the same finite sum and took the same path."""
    outs = _run(what)
    for r in (0, 1):
        out, stats, n_calls = outs[r]
        assert torch.equal(out, torch.full((4, 8), 3.0).to(torch.bfloat16)), (r, out)
        assert stats == {"retries": retries, "fallback_used": fallback, "nan_left": False}
        assert n_calls == 1 + retries
