"""Tensor-parallel and expert-parallel use of the quantized-linear path, one process per GPU over
`torch.distributed` (NCCL on GPUs; the same code runs over gloo in the CPU tests with a stand-in
compute backend).

What the reference does around the ops (vLLM side, `vllm/patches/vllm_for_multi_arc.patch`):
  * column-parallel QKV / gate_up: the N dimension is split, no communication;
  * row-parallel o_proj / down: K is split in multiples of the 128-wide quantisation group, each rank
    produces a full-width partial result and the ranks all-reduce it (`:10185`, `:10199`, `:8006-8010`);
  * expert parallelism: experts are split contiguously over ranks (`:3356-3365`) and tokens are exchanged.
The reference has no fused kernel under EP and emulates all-to-all with all-gather + reduce-scatter
(`:1559-1563`); here tokens really travel by all-to-all with a counts exchange in front.

Only sharding arithmetic and collectives live here; all compute goes through a small backend object so
that the CUDA ops (default) and a CPU oracle (tests) can both drive the same schedule.
"""
from dataclasses import dataclass

import torch
import torch.distributed as dist

GROUP = 128


# ----------------------------------------------------------------------------- sharding of INT4 N-major weights
def shard_column(w: torch.Tensor, scale: torch.Tensor, rank: int, world: int, fused_halves: int = 1):
    """Split output rows.  w [N, K/8] (or [N, K/2]) and scale [N, K/g] are sliced the same way.

    fused_halves = 2 for gate_up: the gate rows and the up rows are each split so that a rank owns matching
    slices ([gate_r ; up_r]); 1 for a plain split (QKV is split by heads by the caller choosing N)."""
    N = w.shape[0]
    assert N % (world * fused_halves) == 0, "N must divide evenly over ranks"
    part = N // fused_halves
    sl = part // world
    rows = torch.cat([torch.arange(h * part + rank * sl, h * part + (rank + 1) * sl) for h in range(fused_halves)])
    rows = rows.to(w.device)
    return w.index_select(0, rows).contiguous(), scale.index_select(0, rows).contiguous()


def shard_row(w: torch.Tensor, scale: torch.Tensor, rank: int, world: int, k_per_word: int = 8):
    """Split the reduction dimension in multiples of the 128-wide group.  w [N, K/k_per_word], scale [N, K/128]."""
    G = scale.shape[1]
    assert G % world == 0, "K/128 must divide evenly over ranks"
    g = G // world
    wcols = g * GROUP // k_per_word
    return (w[:, rank * wcols:(rank + 1) * wcols].contiguous(), scale[:, rank * g:(rank + 1) * g].contiguous())


# ----------------------------------------------------------------------------- compute backends
class CudaBackend:
    """The product path: torch ops of this package (C ABI underneath)."""

    def __init__(self):
        from . import _impl, _lib
        self.I, self.L = _impl, _lib

    def linear_int4(self, x, w, s):
        out = torch.empty(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
        return self.I.linear_int4(x, w, s, out)

    def silu_mul(self, g):
        return self.I.silu_mul(g)

    def topk(self, logits, k, dtype):
        return self.I.moe_topk(logits, k, True, weight_dtype=dtype)

    def route(self, ids, E):
        return self.I.moe_route(ids, E)

    def gather_rows(self, src, idx, div):
        return self.I.gather_rows(src, idx, div)

    def expert_mlp(self, x, w13, s13, w2, s2, offsets, tokens, rows):
        """rows of x (in arrival order) -> y in arrival order, through the experts given by the route."""
        gate_up = self.I.moe_gemm_int4(x, w13, s13, offsets, rows, row_map=tokens, row_div=1)
        return self.I.moe_gemm_int4(gate_up, w2, s2, offsets, rows, out_map=tokens, out_rows=x.shape[0],
                                    act=self.L.ACT_SILU_MUL_IN)

    def combine(self, y, weights, perm, T, k):
        return self.I.moe_combine(y, weights, perm, T, k)


# ----------------------------------------------------------------------------- tensor parallel
@dataclass
class TPLayer:
    """One decoder layer's four INT4 linears, already sharded for this rank."""
    qkv: tuple
    o: tuple
    gate_up: tuple
    down: tuple


def all_reduce(t: torch.Tensor, group=None) -> torch.Tensor:
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def tp_layer_forward(x: torch.Tensor, layer: TPLayer, backend, group=None, reduce=all_reduce, row_linear=None) -> torch.Tensor:
    """x [M, hidden] (replicated) -> [M, hidden] (replicated).

    QKV (column) -> the rank's q slice stands in for the attention output -> o_proj (row, all-reduce)
    -> gate_up (column) -> SiLU*mul -> down (row, all-reduce).  Attention itself is outside this path.
    `reduce(t, group)` sums the partial results over the ranks (default: the process group's all-reduce);
    `row_linear(x, w, s)`, if given, computes a row-parallel linear AND the sum in one call (PeerReducer.row_linear)."""
    qkv = backend.linear_int4(x, *layer.qkv)
    k_local = layer.o[1].shape[1] * GROUP
    attn = qkv[:, :k_local]
    h = row_linear(attn, *layer.o) if row_linear else reduce(backend.linear_int4(attn, *layer.o), group)
    gu = backend.linear_int4(h, *layer.gate_up)
    act = backend.silu_mul(gu)
    return row_linear(act, *layer.down) if row_linear else reduce(backend.linear_int4(act, *layer.down), group)


def _any_nan_globally(t: torch.Tensor, group) -> bool:
    """True on every rank when any rank's tensor holds a NaN (one scalar MAX all-reduce)."""
    flag = torch.isnan(t).any().to(torch.int32).reshape(1)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
    return bool(flag.item())


def guarded_all_reduce(t: torch.Tensor, group=None, max_retries: int = 3, collective=None, stats=None) -> torch.Tensor:
    """All-reduce (sum) with the reference's repair for a collective that returns NaN from finite input
    (vllm/patches/vllm_for_multi_arc.patch:1568-1666): keep a copy of the input; after the collective every rank
    learns through one scalar MAX all-reduce whether ANY rank sees a NaN (all ranks must take the same branch);
    while one does, restore the input and repeat the collective, at most max_retries times; if the NaN is still
    there, restore once more and replace the collective by an all-gather followed by a local sum in rank order
    (:1540-1556).  Off the hot path by design: it costs a clone, a NaN scan and a host round trip per call, so it
    is never the default reduce of tp_layer_forward.  `collective(t, group)` is the in-place sum being guarded
    (default dist.all_reduce); `stats`, if given, receives retries / fallback_used / nan_left."""
    collective = collective or (lambda x, g: dist.all_reduce(x, op=dist.ReduceOp.SUM, group=g))
    if not (dist.is_initialized() and dist.get_world_size(group) > 1) or not t.is_floating_point() or t.numel() == 0:
        return all_reduce(t, group)
    saved = t.clone()
    collective(t, group)
    bad = _any_nan_globally(t, group)
    retries, fallback = 0, False
    while bad and retries < max_retries:
        retries += 1
        t.copy_(saved)
        collective(t, group)
        bad = _any_nan_globally(t, group)
    if bad:
        t.copy_(saved)
        parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, t, group=group)
        t.copy_(parts[0])
        for other in parts[1:]:
            t.add_(other)
        fallback = True
        bad = _any_nan_globally(t, group)
    if stats is not None:
        stats.update(retries=retries, fallback_used=fallback, nan_left=bad)
    return t


class NcclReducer:
    """Sum of row-parallel partial results through the process group's all-reduce (NCCL over NVLink on GPUs)."""

    def reduce(self, t, group=None):
        return all_reduce(t, group)

    def describe(self):
        return "torch.distributed all_reduce (NCCL)"


class PeerReducer:
    """Sum of [M, N] row-parallel partial results through this library's own kernel over peer memory
    (b2q_allreduce_sum in include/b2q.h): one launch per call, plain peer stores over NVLink, bounded flag waits.
    For the decode shapes (M <= 64), where a library all-reduce costs more than the GEMM it follows.

    reduce(t) returns a view of the communicator's result area, valid until the next call but one."""

    def __init__(self, M, N, dtype, device, group=None, mode=0):
        """mode: _lib.COMM_AUTO (one step over the links while a rank sends 8 MiB at most, i.e. for decode tiles; two
        steps beyond), COMM_ONE_STEP or COMM_TWO_STEPS; the same on every rank."""
        import ctypes as C
        from . import _lib as L
        self.L, self.C = L, C
        self.mode = mode
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.M, self.N, self.dtype, self.device = M, N, dtype, torch.device(device)
        self.comm = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        with torch.cuda.device(self.device):
            L.check(L.lib.b2q_comm_create_mode(self.rank, self.world, M, N, mode, C.byref(self.comm), handle))
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.device)
            every = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(every, mine, group=group)
            blob = bytes(torch.cat(every).cpu().tolist())
            L.check(L.lib.b2q_comm_connect(self.comm, blob))
            dist.barrier(group)
        self.views = []
        for which in (0, 1):
            ptr = C.c_void_p()
            L.check(L.lib.b2q_comm_result_ptr(self.comm, which, C.byref(ptr)))
            self.views.append(L.view_as_tensor(ptr.value, (M, N), dtype, self.device, owner=self))
        self.calls = 0

    def reduce(self, t, group=None):
        L, C = self.L, self.C
        if tuple(t.shape) != (self.M, self.N) or t.dtype != self.dtype or t.stride(1) != 1:
            raise RuntimeError("b2q: partial tile does not match the communicator's shape")
        out = C.c_void_p()
        L.check(L.lib.b2q_allreduce_sum(self.comm, t.data_ptr(), L.dt(t), t.stride(0), self.M, self.N, 0.0, C.byref(out),
                                         L.stream(t)))
        view = self.views[self.calls & 1]
        self.calls += 1
        assert view.data_ptr() == out.value
        return view

    def row_linear(self, x, w, s):
        """x [M, K_local] @ dequant(w [N, K_local/8] int32 / [N, K_local/2] uint8, scales s [N, K_local/128])^T summed
        over the ranks, as ONE library call (b2q_linear_int4_allreduce): the GEMM's epilogue delivers its strips
        straight into the owner ranks' reduction slots."""
        from . import _impl as I
        L, C = self.L, self.C
        wt, layout, N, K, sn, sg = I._int4_view(w, s)
        M = x.shape[0]
        if (M, N) != (self.M, self.N) or x.dtype != self.dtype or x.shape[1] != K or x.stride(1) != 1:
            raise RuntimeError("b2q: operands do not match the communicator's tile")
        wsb = L.lib.b2q_linear_workspace_bytes(M, N, K)
        ws = torch.empty(wsb, dtype=torch.uint8, device=x.device)
        partial = torch.empty(M, N, dtype=x.dtype, device=x.device)
        out = C.c_void_p()
        L.check(L.lib.b2q_linear_int4_allreduce(x.data_ptr(), L.dt(x), x.stride(0), wt.data_ptr(), layout, s.data_ptr(), L.dt(s),
                                                 sn, sg, partial.data_ptr(), N, M, N, K, GROUP, L.ptr(ws), wsb, self.comm, 0.0,
                                                 C.byref(out), L.stream(x)))
        view = self.views[self.calls & 1]
        self.calls += 1
        assert view.data_ptr() == out.value
        return view

    def status(self):
        v = self.C.c_int(0)
        self.L.check(self.L.lib.b2q_comm_status(self.comm, self.C.byref(v)))
        return int(v.value)

    def describe(self):
        one = self.mode == 1 or (self.mode == 0 and (self.world - 1) * self.M * self.N * 2 <= (8 << 20))
        form = ("every rank stores its tile into every rank's buffer, every rank adds (one trip over NVLink)" if one else
                "reduce-scatter then broadcast (two trips over NVLink)")
        return "b2q_allreduce_sum: one kernel, plain peer stores, " + form + ", tiles added in rank order (fp32), bounded flag waits"

    def close(self):
        if self.comm:
            self.views = []
            self.L.lib.b2q_comm_destroy(self.comm)
            self.comm = None


class OverlappedReducer:
    """Row-parallel linear + sum for prefill-sized tiles (hundreds of tokens and more), where the sum is bytes, not
    latency: the tokens are cut into chunks, and while the GEMM of chunk i + 1 runs on the caller's stream the
    process group's all-reduce of chunk i runs on a second stream (NCCL over NVLink, a few tens of CTAs).  The weights
    of a rank's shard are re-read once per chunk (from L2 where the shard fits).  The results are those of the
    unchunked form: every output row depends on its own token only and the all-reduce adds the same values.
    Measured on the Llama-70B-shape layer at 2048 tokens: level with the plain all-reduce on two GPUs (1970 against
    1994 us per layer), slower on four and eight (1490 against 1223, 1169 against 930): 512-token GEMMs run at a lower
    rate than one 2048-token GEMM and the all-reduce's CTAs take SMs from them.  Split by output columns instead (all
    tokens per piece, full token tiles) it measured 1909 us with two pieces and 2164 with four against 1815 for the plain
    all-reduce on the same two GPUs.  Opt-in only."""

    def __init__(self, chunks=4, min_chunk_rows=256, group=None, split="tokens"):
        """split = "tokens": chunks of rows of x (every chunk re-reads the weight shard); "columns": chunks of output
        columns, i.e. of weight rows (every chunk keeps all tokens, so the GEMM's token tiles stay full; the pieces are
        joined by one copy at the end)."""
        from . import _impl
        self.I, self.group = _impl, group
        self.chunks, self.min_rows, self.split = int(chunks), int(min_chunk_rows), split
        self.side = torch.cuda.Stream()

    def reduce(self, t, group=None):
        return all_reduce(t, group if group is not None else self.group)

    def row_linear(self, x, w, s):
        M, N = x.shape[0], w.shape[0]
        main = torch.cuda.current_stream(x.device)
        if self.split == "columns":
            step = -(-N // self.chunks)
            step = (step + 127) // 128 * 128                      # whole strips of 128 weight rows
            parts = []
            for lo in range(0, N, step):
                part = torch.empty(M, min(step, N - lo), dtype=x.dtype, device=x.device)
                self.I.linear_int4(x, w[lo:lo + step], s[lo:lo + step], part)
                done = torch.cuda.Event()
                done.record(main)
                self.side.wait_event(done)
                with torch.cuda.stream(self.side):
                    dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
                parts.append(part)
            main.wait_stream(self.side)
            return torch.cat(parts, dim=1)
        out = torch.empty(M, N, dtype=x.dtype, device=x.device)
        step = max(self.min_rows, -(-M // self.chunks))
        for lo in range(0, M, step):
            part = out[lo:lo + step]
            self.I.linear_int4(x[lo:lo + step], w, s, part)
            done = torch.cuda.Event()
            done.record(main)
            self.side.wait_event(done)
            with torch.cuda.stream(self.side):
                dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
        main.wait_stream(self.side)            # also keeps `out` from being reused before the second stream is done
        return out

    def describe(self):
        return ("torch.distributed all_reduce (NCCL) per chunk of %d tokens at least, on a second stream under the GEMM "
                "of the next chunk" % self.min_rows)


def make_reducer(M, N, dtype, device, group=None, kind=None, mode=0):
    """The object whose reduce(t) sums a [M, N] partial result over the ranks of `group`: this library's peer-memory
    kernel for decode-sized tiles on CUDA devices, the process group's all-reduce otherwise (kind / B2Q_REDUCER =
    "peer", "nccl" or "overlap" forces one; "overlap" = OverlappedReducer, which measured slower than the plain
    all-reduce on 4 and 8 GPUs and is therefore never chosen by default)."""
    import os
    kind = kind or os.environ.get("B2Q_REDUCER")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    cuda = torch.device(device).type == "cuda"
    if kind is None:
        if cuda and world > 1 and world <= 8 and M <= 64 and N % (8 * world) == 0:
            kind = "peer"
        else:
            kind = "nccl"
    if kind == "peer" and cuda and world > 1:
        return PeerReducer(M, N, dtype, device, group, mode)
    if kind == "overlap" and cuda and world > 1:
        return OverlappedReducer(group=group)
    return NcclReducer()


# ----------------------------------------------------------------------------- expert parallel
def ep_plan(ids: torch.Tensor, experts_per_rank: int, world: int, backend):
    """Sort this rank's (token, slot) pairs by destination rank.

    Returns send_counts [world] (host list), send_order int32 [n_pairs] (pair indices grouped by destination,
    stable), pair_to_send int32 [n_pairs] (inverse), local_expert int32 [n_pairs] in send order."""
    dest = torch.div(ids, experts_per_rank, rounding_mode="floor").to(torch.int32).contiguous()
    offsets, order, p2s, rows = backend.route(dest, world)
    local_e = (ids.reshape(-1) % experts_per_rank).to(torch.int32)[order.long()].contiguous()
    return rows.tolist(), order, p2s, local_e


EP_EXCHANGE = "torch.distributed all_to_all_single (NCCL send/recv), row counts read on the host"


class EpExchange:
    """Token exchange of the expert-parallel layer through this library's own kernels over peer memory (b2q_ep_* in
    include/b2q.h): rows go to their experts' ranks and results come back by plain peer stores, every count stays on
    the device, so a pass has no host read and no stalled stream.  cap_rows = this rank's tokens x top_k (the same on
    every rank), H = row width."""

    def __init__(self, cap_rows, H, dtype, device, group=None):
        import ctypes as C
        from . import _lib as L
        self.L, self.C = L, C
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.cap, self.H, self.dtype, self.device = int(cap_rows), int(H), dtype, torch.device(device)
        self.comm = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        with torch.cuda.device(self.device):
            L.check(L.lib.b2q_ep_create(self.rank, self.world, self.cap, self.H, C.byref(self.comm), handle))
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.device)
            every = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(every, mine, group=group)
            L.check(L.lib.b2q_ep_connect(self.comm, bytes(torch.cat(every).cpu().tolist())))
            dist.barrier(group)
        self._views()

    def _views(self):
        L, C = self.L, self.C
        rows, ids, ret = C.c_void_p(), C.c_void_p(), C.c_void_p()
        L.check(L.lib.b2q_ep_buffers(self.comm, C.byref(rows), C.byref(ids), C.byref(ret)))
        n = self.world * self.cap
        self.recv_rows = L.view_as_tensor(rows.value, (n, self.H), self.dtype, self.device, owner=self)
        self.recv_ids = L.view_as_tensor(ids.value, (n,), torch.int32, self.device, owner=self)
        self.ret_rows = L.view_as_tensor(ret.value, (self.cap, self.H), self.dtype, self.device, owner=self)

    def dispatch(self, x, order, top_k, dest_offsets, local_ids):
        L = self.L
        L.check(L.lib.b2q_ep_dispatch(self.comm, x.data_ptr(), L.dt(x), x.stride(0), order.data_ptr(), top_k,
                                       dest_offsets.data_ptr(), local_ids.data_ptr(), order.numel(), L.stream(x)))

    def wait(self, phase, like):
        self.L.check(self.L.lib.b2q_ep_wait(self.comm, phase, 0.0, self.L.stream(like)))

    def give_back(self, y):
        L = self.L
        L.check(L.lib.b2q_ep_return(self.comm, y.data_ptr(), L.dt(y), y.stride(0), L.stream(y)))

    def status(self):
        v = self.C.c_int(0)
        self.L.check(self.L.lib.b2q_ep_status(self.comm, self.C.byref(v)))
        return v.value

    def describe(self):
        return ("b2q_ep_dispatch / b2q_ep_return: rows and results by plain peer stores over NVLink into fixed-capacity "
                "slots, counts and offsets exchanged as data, bounded flag waits, no host read per pass")

    def close(self):
        if self.comm:
            self.recv_rows = self.recv_ids = self.ret_rows = None
            self.L.lib.b2q_ep_destroy(self.comm)
            self.comm = None


def ep_moe_forward_device(x, logits, w13, s13, w2, s2, top_k: int, num_experts: int, backend, exchange, marks=None):
    """ep_moe_forward with the exchange done by `exchange` (EpExchange): the same steps, no count ever read on the
    host.  The owner runs its grouped GEMMs over the whole receive area (world x cap rows as an upper bound); the
    counting sort drops the empty positions and the kernels take the row count from its last offset."""
    mark = marks if marks is not None else (lambda label: None)
    world = exchange.world
    T, H = x.shape
    e_local = num_experts // world
    wts, ids = backend.topk(logits, top_k, x.dtype)
    dest = torch.div(ids, e_local, rounding_mode="floor").to(torch.int32).contiguous()
    offsets, order, p2s, _ = backend.route(dest, world)
    local_e = (ids.reshape(-1) % e_local).to(torch.int32)[order.long()].contiguous()
    mark("dispatch_begin")
    exchange.dispatch(x, order, top_k, offsets, local_e)
    exchange.wait(0, x)
    mark("dispatch_end")
    n = world * exchange.cap
    r_off, r_tok, _, _ = backend.route(exchange.recv_ids.reshape(-1, 1), e_local)
    y = backend.expert_mlp(exchange.recv_rows, w13, s13, w2, s2, r_off, r_tok, n)
    mark("combine_begin")
    exchange.give_back(y)
    exchange.wait(1, x)
    mark("combine_end")
    return backend.combine(exchange.ret_rows[:T * top_k], wts, p2s, T, top_k)


def ep_moe_forward(x, logits, w13, s13, w2, s2, top_k: int, num_experts: int, backend, group=None, marks=None, world=None):
    """Expert-parallel MoE forward for this rank's tokens.

    x [T_local, H], logits [T_local, E]; w13 / s13 / w2 / s2 hold this rank's experts
    [E/world, ...].  Steps: top-k -> plan by destination rank -> exchange counts -> all-to-all rows and
    local expert ids -> route + grouped up GEMM + SiLU*mul + grouped down GEMM on the owner -> all-to-all back
    -> weighted combine at the source.  Returns [T_local, H].
    `marks`, if given, is called with a label at the phase boundaries (a benchmark records CUDA events there)."""
    mark = marks if marks is not None else (lambda label: None)
    if world is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
    T, H = x.shape
    e_local = num_experts // world
    wts, ids = backend.topk(logits, top_k, x.dtype)
    send_counts, order, p2s, local_e = ep_plan(ids, e_local, world, backend)
    send_rows = backend.gather_rows(x, order, top_k)                       # [n_pairs, H] grouped by destination
    mark("dispatch_begin")

    if world > 1:
        sc = torch.tensor(send_counts, dtype=torch.int64, device=x.device)
        rc = torch.empty_like(sc)
        dist.all_to_all_single(rc, sc, group=group)
        recv_counts = rc.tolist()
        n_recv = int(sum(recv_counts))
        recv_rows = torch.empty(n_recv, H, dtype=x.dtype, device=x.device)
        recv_e = torch.empty(n_recv, dtype=torch.int32, device=x.device)
        dist.all_to_all_single(recv_rows, send_rows, recv_counts, send_counts, group=group)
        dist.all_to_all_single(recv_e, local_e, recv_counts, send_counts, group=group)
    else:
        recv_counts, n_recv, recv_rows, recv_e = send_counts, send_rows.shape[0], send_rows, local_e

    mark("dispatch_end")
    if n_recv > 0:
        offsets, tokens, _, _ = backend.route(recv_e.reshape(-1, 1), e_local)
        y_recv = backend.expert_mlp(recv_rows, w13, s13, w2, s2, offsets, tokens, n_recv)
    else:
        y_recv = torch.empty(0, H, dtype=x.dtype, device=x.device)

    mark("combine_begin")
    if world > 1:
        y_send = torch.empty(send_rows.shape[0], H, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(y_send, y_recv, send_counts, recv_counts, group=group)
    else:
        y_send = y_recv
    mark("combine_end")
    return backend.combine(y_send, wts, p2s, T, top_k)
