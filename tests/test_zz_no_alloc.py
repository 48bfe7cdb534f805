"""The workspace-free routing entry point (b2q_moe_route_static).

Some users of this library cannot allocate device memory around a call: they run inside a CUDA stream
capture, or their runtime has handed out all device memory before the first token arrives.  For them
the routing sort keeps its scratch table in a fixed array inside the library.  This test drives that
entry point through the C ABI, twice in a row, and requires exactly the outputs of the ordinary
b2q_moe_route (integer work: bit-exact).  The file name sorts last so that a run stopping at the first
failure has already been through every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def L(lib_built):
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    from custom_esimd_kernels_vllm import _lib
    return _lib


def _route_both(L, ids, E):
    n = ids.numel()
    dev = ids.device
    outs = []
    for static in (False, True):
        off = torch.full((E + 1,), -7, dtype=torch.int32, device=dev)
        tok = torch.full((n,), -7, dtype=torch.int32, device=dev)
        p2p = torch.full((n,), -7, dtype=torch.int32, device=dev)
        rows = torch.full((E,), -7, dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        if static:
            rc = L.lib.b2q_moe_route_static(ids.data_ptr(), n, E, off.data_ptr(), tok.data_ptr(), p2p.data_ptr(),
                                            rows.data_ptr(), stream)
        else:
            wsb = L.lib.b2q_moe_route_workspace_bytes(n, E)
            ws = torch.empty(wsb, dtype=torch.uint8, device=dev)
            rc = L.lib.b2q_moe_route(ids.data_ptr(), n, E, off.data_ptr(), tok.data_ptr(), p2p.data_ptr(),
                                     rows.data_ptr(), ws.data_ptr(), wsb, stream)
        assert rc == 0, L.lib.b2q_strerror(rc)
        torch.cuda.synchronize()
        outs.append((off.cpu(), tok.cpu(), p2p.cpu(), rows.cpu()))
    return outs


def test_static_route_matches_workspace_route_on_two_calls_in_a_row(L):
    g = torch.Generator().manual_seed(42)
    # two different problems back to back: the second must not see anything of the first in the shared table
    for T, k, E in ((4096, 8, 128), (777, 4, 256)):
        ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
        ids[ids == 3] = 5                      # an expert without rows
        ids[0, 0] = E + 9                      # one pair routed to an expert this rank does not own
        ref, got = _route_both(L, ids.to(DEV), E)
        for a, b in zip(ref, got):
            assert torch.equal(a, b)
        assert int(ref[0][-1]) == T * k - 1


def test_static_route_rejects_sizes_beyond_its_table(L):
    ids = torch.zeros(8, dtype=torch.int32, device=DEV)
    out = torch.zeros(2048, dtype=torch.int32, device=DEV)
    p = out.data_ptr()
    assert L.lib.b2q_moe_route_static(ids.data_ptr(), 65537, 8, p, p, p, p, None) == -10
    assert L.lib.b2q_moe_route_static(ids.data_ptr(), 8, 257, p, p, p, p, None) == -10
    assert L.lib.b2q_strerror(-10).startswith(b"b2q:")
    assert L.lib.b2q_moe_route_static(None, 8, 8, p, p, p, p, None) == -1


@pytest.mark.gpu
def test_route_static_inside_a_stream_capture_and_on_a_second_device(lib_built):
    """The stated use: one eager call per device, then the routing sort captured into a CUDA graph on a side stream
    and replayed with different ids; every replay must equal b2q_moe_route bit for bit.  With two GPUs visible the
    eager comparison is repeated on cuda:1 (the scratch table's address is looked up per device)."""
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    import custom_esimd_kernels_vllm as pkg
    L, I = pkg._lib, pkg._impl
    E, n = 32, 4096

    def static_route(ids, outs, stream):
        L.check(L.lib.b2q_moe_route_static(ids.data_ptr(), n, E, outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(),
                                            outs[3].data_ptr(), stream.cuda_stream))

    for dev in range(min(2, torch.cuda.device_count())):
        d = torch.device("cuda", dev)
        with torch.cuda.device(d):
            g = torch.Generator(device=d).manual_seed(dev)
            ids = torch.randint(0, E, (n, 1), generator=g, device=d, dtype=torch.int32)
            outs = [torch.empty(E + 1, dtype=torch.int32, device=d), torch.empty(n, dtype=torch.int32, device=d),
                    torch.empty(n, dtype=torch.int32, device=d), torch.empty(E, dtype=torch.int32, device=d)]
            static_route(ids, outs, torch.cuda.current_stream())              # the first call on this device, eager
            torch.cuda.synchronize()
            for got, want in zip(outs, I.moe_route(ids, E)):
                assert torch.equal(got, want)
            if dev > 0:
                continue
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    static_route(ids, outs, side)
            for rep in range(2):
                ids.copy_(torch.randint(0, E, (n, 1), generator=g, device=d, dtype=torch.int32))
                for o in outs:
                    o.fill_(-7)
                torch.cuda.synchronize()
                graph.replay()
                torch.cuda.synchronize()
                for got, want in zip(outs, I.moe_route(ids, E)):
                    assert torch.equal(got, want), rep
