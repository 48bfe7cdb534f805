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
