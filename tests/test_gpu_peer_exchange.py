"""The expert-parallel token exchange over peer memory (b2q_ep_*), on ONE GPU.

All ranks live in this process on one device (b2q_ep_connect_local): the same kernels, slots, flags and pass
numbers as the multi-GPU path, with the peer pointers pointing at buffers of the same device.  Every step runs for
all ranks before the next step begins, so no kernel ever waits for a later launch.  Rows must arrive at their
owners in the order of the source's destination sort, empty slot positions must carry the index -1, and the
results must come back at the positions of the source's send order, bit for bit, over several passes on the same
buffers.  The give-up path is exercised with a rank that never sends: the wait runs out after a millisecond,
the code is readable from the host and the context stays usable.  Nothing faults or hangs.
"""
import ctypes as C

import pytest
import torch

from gpu_util import DEV

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg(lib_built):
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    import custom_esimd_kernels_vllm as e
    return e


class Ranks:
    def __init__(self, L, world, cap, H, dtype=torch.bfloat16):
        self.L, self.world, self.cap, self.H = L, world, cap, H
        self.comms = (C.c_void_p * world)()
        for r in range(world):
            c = C.c_void_p()
            L.check(L.lib.b2q_ep_create(r, world, cap, H, C.byref(c), None))
            self.comms[r] = c
        L.check(L.lib.b2q_ep_connect_local(self.comms, world))
        self.recv_rows, self.recv_ids, self.ret_rows = [], [], []
        for r in range(world):
            a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
            L.check(L.lib.b2q_ep_buffers(self.comms[r], C.byref(a), C.byref(b), C.byref(c)))
            self.recv_rows.append(L.view_as_tensor(a.value, (world * cap, H), dtype, torch.device(DEV)))
            self.recv_ids.append(L.view_as_tensor(b.value, (world * cap,), torch.int32, torch.device(DEV)))
            self.ret_rows.append(L.view_as_tensor(c.value, (cap, H), dtype, torch.device(DEV)))

    def stream(self):
        return torch.cuda.current_stream().cuda_stream

    def dispatch(self, r, x, order, k, offsets, local_ids):
        L = self.L
        L.check(L.lib.b2q_ep_dispatch(self.comms[r], x.data_ptr(), L.dt(x), x.stride(0), order.data_ptr(), k, offsets.data_ptr(),
                                       local_ids.data_ptr(), order.numel(), self.stream()))

    def wait(self, r, phase, limit_ms=0.0):
        self.L.check(self.L.lib.b2q_ep_wait(self.comms[r], phase, C.c_double(limit_ms), self.stream()))

    def give_back(self, r, y):
        L = self.L
        L.check(L.lib.b2q_ep_return(self.comms[r], y.data_ptr(), L.dt(y), y.stride(0), self.stream()))

    def status(self, r=0):
        v = C.c_int(0)
        self.L.check(self.L.lib.b2q_ep_status(self.comms[r], C.byref(v)))
        return v.value

    def close(self):
        self.recv_rows = self.recv_ids = self.ret_rows = None
        for r in range(self.world):
            self.L.lib.b2q_ep_destroy(self.comms[r])


@pytest.mark.parametrize("world,T,k,H,E", [(2, 64, 2, 256, 8), (4, 48, 4, 512, 16), (8, 33, 8, 2048, 128), (3, 7, 1, 64, 6)])
def test_rows_reach_their_owners_and_results_come_back(pkg, world, T, k, H, E):
    L, I = pkg._lib, pkg._impl
    e_local = E // world
    ranks = Ranks(L, world, T * k, H)
    try:
        g = torch.Generator(device=DEV).manual_seed(world * 100 + T)
        for rnd in range(3):                                   # three passes on the same buffers, nothing cleared
            xs = [torch.randn(T, H, generator=g, device=DEV).to(torch.bfloat16) for _ in range(world)]
            ids = [torch.randint(0, E, (T, k), generator=g, device=DEV, dtype=torch.int32) for _ in range(world)]
            if rnd == 1:
                ids[0][:] = E - 1                              # one rank sends everything to the last owner
            plans = []
            for r in range(world):
                dest = torch.div(ids[r], e_local, rounding_mode="floor").to(torch.int32).contiguous()
                offsets, order, p2s, _ = I.moe_route(dest, world)
                local = (ids[r].reshape(-1) % e_local).to(torch.int32)[order.long()].contiguous()
                plans.append((offsets, order, local))
                ranks.dispatch(r, xs[r], order, k, offsets, local)
            for r in range(world):
                ranks.wait(r, 0)
            torch.cuda.synchronize()
            # what every owner must hold: slot s = the rows source s sorted to it, in order, then -1
            for j in range(world):
                for s in range(world):
                    offsets, order, local = plans[s]
                    lo, hi = int(offsets[j]), int(offsets[j + 1])
                    slot = slice(s * T * k, s * T * k + (hi - lo))
                    want_rows = xs[s][(order[lo:hi] // k).long()]
                    assert torch.equal(ranks.recv_rows[j][slot], want_rows), (rnd, j, s)
                    assert torch.equal(ranks.recv_ids[j][slot], local[lo:hi]), (rnd, j, s)
                    rest = ranks.recv_ids[j][s * T * k + (hi - lo):(s + 1) * T * k]
                    assert bool((rest == -1).all()), (rnd, j, s)
            # the owners' "results": twice the row where a row arrived
            for j in range(world):
                y = torch.where((ranks.recv_ids[j] >= 0).unsqueeze(1), ranks.recv_rows[j] * 2, torch.full_like(ranks.recv_rows[j], 77.0))
                ranks.give_back(j, y)
            for r in range(world):
                ranks.wait(r, 1)
            torch.cuda.synchronize()
            for r in range(world):
                _, order, _ = plans[r]
                want = xs[r][(order // k).long()] * 2
                assert torch.equal(ranks.ret_rows[r][:T * k], want), (rnd, r)
        assert all(ranks.status(r) == 0 for r in range(world))
    finally:
        ranks.close()


def test_absent_rank_makes_the_wait_give_up_and_report(pkg):
    L, I = pkg._lib, pkg._impl
    ranks = Ranks(L, 2, 32, 64)
    try:
        x = torch.ones(16, 64, dtype=torch.bfloat16, device=DEV)
        ids = torch.zeros(16, 2, dtype=torch.int32, device=DEV)
        offsets, order, _, _ = I.moe_route(ids, 2)
        ranks.dispatch(0, x, order, 2, offsets, torch.zeros(32, dtype=torch.int32, device=DEV))
        ranks.wait(0, 0, limit_ms=1.0)                         # rank 1 never sends
        torch.cuda.synchronize()
        assert ranks.status(0) == 301
    finally:
        ranks.close()
    ranks = Ranks(L, 2, 32, 64)                                # the context is intact
    try:
        assert ranks.status(0) == 0
    finally:
        ranks.close()


def test_rejects_shapes_outside_the_contract(pkg):
    L = pkg._lib
    c = C.c_void_p()
    assert L.lib.b2q_ep_create(0, 9, 64, 256, C.byref(c), None) != 0           # more ranks than one box holds
    assert L.lib.b2q_ep_create(0, 2, 64, 250, C.byref(c), None) != 0           # rows not a multiple of 16 bytes
    ranks = Ranks(L, 2, 16, 64)
    try:
        x = torch.zeros(16, 64, dtype=torch.bfloat16, device=DEV)
        order = torch.zeros(32, dtype=torch.int32, device=DEV)
        off = torch.zeros(3, dtype=torch.int32, device=DEV)
        with pytest.raises(RuntimeError):
            ranks.dispatch(0, x, order, 2, off, order)                          # more pairs than a slot holds
    finally:
        ranks.close()
