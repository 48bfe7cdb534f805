"""Host-side classification of INT4 weight presentations (no device needed)."""
import pytest
import torch

from oracle import int4


@pytest.fixture(scope="module")
def impl(lib_built):
    from custom_esimd_kernels_vllm import _impl, _lib
    return _impl, _lib


def test_int4_view_accepts_every_reference_presentation(impl):
    I, L = impl
    N, K = 48, 256
    q = torch.randint(0, 16, (N, K), dtype=torch.uint8)
    s = torch.rand(N, K // 128).to(torch.bfloat16)
    w32 = int4.pack_nmajor_i32(q)
    u8 = int4.pack_nmajor_u8(q)
    # uint8 [N, K/2]
    wt, lay, n, k, sn, sg = I._int4_view(u8, s)
    assert (lay, n, k, sn, sg) == (L.W4_NMAJOR, N, K, K // 128, 1)
    # int32 [N, K/8]
    assert I._int4_view(w32, s)[1:4] == (L.W4_NMAJOR, N, K)
    # the GPTQ view: qweight.t() aliasing the same bytes, scales .t().contiguous()
    st = s.t().contiguous()
    wt, lay, n, k, sn, sg = I._int4_view(w32.t(), st)
    assert (lay, n, k, sn, sg) == (L.W4_NMAJOR, N, K, 1, N)
    assert wt.data_ptr() == w32.data_ptr() and wt.is_contiguous()
    # materialised contiguous [K/8, N]
    wk, sk = int4.to_kmajor(w32, s, marlin=False)
    wt, lay, n, k, sn, sg = I._int4_view(wk, sk)
    assert (lay, n, k, sn, sg) == (L.W4_KMAJOR, N, K, 1, N)


def test_int4_view_rejects_bad_shapes(impl):
    I, _ = impl
    with pytest.raises(RuntimeError):
        I._int4_view(torch.zeros(8, 20, dtype=torch.uint8), torch.zeros(8, 1))       # K = 40 not a group multiple
    with pytest.raises(RuntimeError):
        I._int4_view(torch.zeros(8, 64, dtype=torch.uint8), torch.zeros(8, 3))       # scale shape
    with pytest.raises(RuntimeError):
        I._int4_view(torch.zeros(8, 64, dtype=torch.int16), torch.zeros(8, 1))       # dtype


def test_python_repack_helpers_match_oracle(impl):
    import custom_esimd_kernels_vllm as e
    q = torch.randint(0, 16, (3, 16, 256), dtype=torch.uint8)
    w32 = int4.pack_nmajor_i32(q)
    u8 = e.to_cutlass_nmajor_int4(w32)
    assert torch.equal(u8, int4.pack_nmajor_u8(q))
    assert torch.equal(e.cutlass_nmajor_int4_to_signed(u8), int4.u4_to_s4_bytes(u8))
    w, ids = torch.rand(5, 2), torch.randint(0, 4, (5, 2), dtype=torch.int32)
    rows, wts, per = e.precompute_moe_route(w, ids, 4)     # CPU tensors take the torch fallback
    assert per.sum() == 10 and rows.numel() == 10
