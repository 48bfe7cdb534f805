"""The peer-memory sum of row-parallel partial results (b2q_allreduce_sum), on ONE GPU.

All ranks of the protocol live in this process on one device and run as a single cooperative launch
(b2q_allreduce_sum_emulated): the same kernel, flags, epochs and buffer layout as the multi-GPU path, with the
peer pointers pointing at buffers of the same device.  Ranks that wait for one another are never run as separate
launches on one GPU.  The sums must be bit-identical to adding the partial tiles in rank order in fp32.
The give-up path is exercised with a rank that never arrives: the present rank's wait runs out after a
millisecond, the code is readable from the host and the context stays usable.  Nothing faults or hangs.
"""
import ctypes as C

import pytest
import torch

from gpu_util import DEV

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L(lib_built):
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    import custom_esimd_kernels_vllm as pkg
    return pkg._lib


class Ranks:
    def __init__(self, L, world, M, N, mode=0):
        self.L, self.world, self.M, self.N = L, world, M, N
        self.comms = (C.c_void_p * world)()
        for r in range(world):
            c = C.c_void_p()
            L.check(L.lib.b2q_comm_create_mode(r, world, M, N, mode, C.byref(c), None))
            self.comms[r] = c
        L.check(L.lib.b2q_comm_connect_local(self.comms, world))

    def reduce(self, ins, present=None, limit_ms=0.0):
        L, n = self.L, present or self.world
        ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in ins[:n]])
        outs = (C.c_void_p * n)()
        t0 = ins[0]
        rc = L.lib.b2q_allreduce_sum_emulated(self.comms, self.world, n, ptrs, L.dt(t0), t0.stride(0), t0.shape[0], t0.shape[1],
                                              C.c_double(limit_ms), outs, torch.cuda.current_stream().cuda_stream)
        L.check(rc)
        return [L.view_as_tensor(outs[r], tuple(t0.shape), t0.dtype, t0.device) for r in range(n)]

    def status(self, r=0):
        v = C.c_int(0)
        self.L.check(self.L.lib.b2q_comm_status(self.comms[r], C.byref(v)))
        return v.value

    def close(self):
        for r in range(self.world):
            self.L.lib.b2q_comm_destroy(self.comms[r])


def _ordered_sum(ins):
    acc = torch.zeros_like(ins[0], dtype=torch.float32)
    for t in ins:
        acc += t.float()
    return acc.to(ins[0].dtype)


@pytest.mark.parametrize("world,M,N,dtype", [(2, 64, 8192, torch.bfloat16), (4, 64, 8192, torch.bfloat16), (8, 64, 8192, torch.bfloat16),
                                             (4, 7, 768, torch.float16), (8, 1, 1024, torch.bfloat16), (3, 16, 1200, torch.float16)])
@pytest.mark.parametrize("mode", [1, 2])           # one step over the links / two steps (reduce-scatter, broadcast)
def test_sum_is_bit_identical_to_rank_order_fp32(L, world, M, N, dtype, mode):
    ranks = Ranks(L, world, M, N, mode)
    try:
        g = torch.Generator(device=DEV).manual_seed(world * 1000 + M)
        for call in range(5):                    # several epochs on the same buffers (both slot sets), nothing cleared in between
            ins = [torch.randn(M, N, generator=g, device=DEV).to(dtype) for _ in range(world)]
            outs = ranks.reduce(ins)
            torch.cuda.synchronize()
            ref = _ordered_sum(ins)
            for r in range(world):
                assert torch.equal(outs[r], ref), (call, r)
        assert ranks.status() == 0
    finally:
        ranks.close()


@pytest.mark.parametrize("mode", [0, 2])
def test_row_pitch_and_smaller_tile_than_the_bound(L, mode):
    ranks = Ranks(L, 4, 64, 8192, mode)
    try:
        g = torch.Generator(device=DEV).manual_seed(5)
        wide = [torch.randn(40, 4096 + 64, generator=g, device=DEV).to(torch.bfloat16) for _ in range(4)]
        ins = [w[:, :4096] for w in wide]                        # row pitch 4160, tile smaller than the communicator's bound
        outs = ranks.reduce(ins)
        torch.cuda.synchronize()
        assert torch.equal(outs[2], _ordered_sum(ins))
    finally:
        ranks.close()


@pytest.mark.parametrize("mode", [1, 2])
def test_absent_rank_makes_the_wait_give_up_and_report(L, mode):
    ranks = Ranks(L, 2, 16, 1024, mode)
    x = [torch.ones(16, 1024, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    try:
        ranks.reduce(x, present=1, limit_ms=1.0)                 # rank 1 never arrives
        torch.cuda.synchronize()
        assert ranks.status(0) == 201                            # the wait for the partial blocks ran out
    finally:
        ranks.close()
    # the context is intact: a fresh set of communicators works
    ranks = Ranks(L, 2, 16, 1024, mode)
    try:
        outs = ranks.reduce(x)
        torch.cuda.synchronize()
        assert torch.equal(outs[0], x[0] * 2) and ranks.status(0) == 0
    finally:
        ranks.close()


def test_rejects_shapes_outside_the_contract(L):
    c = C.c_void_p()
    assert L.lib.b2q_comm_create(0, 9, 64, 8192, C.byref(c), None) != 0          # more ranks than one box holds
    assert L.lib.b2q_comm_create(0, 4, 64, 8190, C.byref(c), None) != 0          # N not a multiple of 8 * world
    ranks = Ranks(L, 2, 16, 1024)
    try:
        big = [torch.zeros(32, 1024, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
        with pytest.raises(RuntimeError):
            ranks.reduce(big)                                                    # more rows than the communicator was made for
    finally:
        ranks.close()
