"""Oracle checks on SLICES of full-size problems (test infrastructure only, like the rest of this package).

The benchmark configurations are too large to push through a CPU matmul in full (config 3 is 0.73 TFLOP,
one decoder layer of config 5 at 2048 tokens is 3.5 TFLOP), but every output element of a linear layer
depends on one activation row and one weight row only, and every output row of the MoE pipeline on one token
only.  A slice of the oracle is therefore exact: these helpers take the tensors a GPU run used (any device),
copy the rows a seeded selection names to the CPU, run the functions of oracle.int4 / oracle.fp8 / oracle.moe
on them and return the error of the matching slice of the GPU result, in the forms the reference's tests
report (tests/test_gemv_int4.py:463-466, :595; tests/test_fp8_blockscale_gemm.py:53-59).
"""
import torch

from . import fp8, int4, moe


def errors(out: torch.Tensor, ref: torch.Tensor) -> dict:
    o, r = out.detach().float().cpu(), ref.detach().float().cpu()
    d = (o - r).abs()
    mx = float(r.abs().max().clamp(min=1e-30))
    return {"max_rel_err": float(d.max()) / mx,
            "mean_rel_err": float(d.mean() / r.abs().mean().clamp(min=1e-30)),
            "cos": float(torch.nn.functional.cosine_similarity(o.flatten().double(), r.flatten().double(), dim=0))}


def pick(n: int, count: int, seed: int, every: int = 0) -> torch.Tensor:
    """Sorted seeded selection of `count` indices below n; with `every` > 0 additionally one index out of every
    block of `every` consecutive ones (so that each 128-row strip / token tile of a kernel contributes)."""
    g = torch.Generator().manual_seed(seed)
    idx = torch.randperm(n, generator=g)[:min(count, n)]
    if every > 0:
        blocks = torch.arange(0, n, every)
        off = torch.randint(0, every, (blocks.numel(),), generator=g)
        idx = torch.cat([idx, (blocks + off).clamp(max=n - 1)])
    return torch.unique(idx)


def _rows(t: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    return t.index_select(0, idx.to(t.device)).cpu()


def int4_linear(x, w_i32, scale, out, cols=None, toks=None):
    """out[toks][:, cols] against oracle.int4.linear for an N-major int32 [N, K/8] weight with scales [N, K/128]."""
    N = w_i32.shape[0]
    cols = torch.arange(N) if cols is None else cols
    toks = torch.arange(x.shape[0]) if toks is None else toks
    q = int4.unpack_nmajor_i32(_rows(w_i32, cols))
    ref = int4.linear(_rows(x, toks), q, _rows(scale, cols))
    got = _rows(out, toks)[:, cols]
    return errors(got, ref.to(out.dtype))


def fp8_channel_linear(x, wq, scale, out, cols=None, toks=None):
    N = wq.shape[0]
    cols = torch.arange(N) if cols is None else cols
    toks = torch.arange(x.shape[0]) if toks is None else toks
    ref = fp8.linear_channel(_rows(x, toks), _rows(wq.view(torch.uint8), cols), _rows(scale.reshape(-1, 1), cols).reshape(-1))
    return errors(_rows(out, toks)[:, cols], ref.to(out.dtype))


def _block_rows(wq, ws, cols):
    """Dequantised rows `cols` of a 128x128 block-scaled e4m3 weight (fp32 [len(cols), K])."""
    K = wq.shape[1]
    s = _rows(ws, torch.div(cols, 128, rounding_mode="floor")).repeat_interleave(128, dim=1)[:, :K]
    return fp8.decode(_rows(wq.view(torch.uint8), cols)) * s


def fp8_block_w8a16(x, wq, ws, out, cols, toks):
    ref = _rows(x, toks).float() @ _block_rows(wq, ws, cols).T
    return errors(_rows(out, toks)[:, cols], ref.to(out.dtype))


def fp8_block_w8a8(xq, xs, wq, ws, out, cols, toks):
    a = fp8.dequant_act_1x128(_rows(xq.view(torch.uint8), toks), _rows(xs, toks))
    ref = a @ _block_rows(wq, ws, cols).T
    return errors(_rows(out, toks)[:, cols], ref.to(out.dtype))


def dequant_experts(w_i32, scale, dtype):
    """[E, N, K/8] int32 + [E, N, K/128] scales -> dequantised [E, N, K] in dtype, one expert at a time."""
    w, s = w_i32.cpu(), scale.cpu()
    return torch.stack([int4.dequant(int4.unpack_nmajor_i32(w[e]), s[e], dtype) for e in range(w.shape[0])])


class LazyExperts:
    """Stands in for a dequantised [E, N, K] tensor in oracle.moe.forward: expert e is fetched from the device and
    dequantised the first time it is indexed, so a check on a few tokens touches only the experts they route to."""

    def __init__(self, w_i32, scale, dtype):
        self.w, self.s, self.dtype, self.cache = w_i32, scale, dtype, {}
        self.shape = (w_i32.shape[0], w_i32.shape[1], w_i32.shape[2] * 8)

    def __getitem__(self, e):
        if e not in self.cache:
            self.cache[e] = int4.dequant(int4.unpack_nmajor_i32(self.w[e].cpu()), self.s[e].cpu(), self.dtype)
        return self.cache[e]


def moe_int4(x, logits, w13_i32, s13, w2_i32, s2, top_k, out, toks, experts=None):
    """Rows `toks` of the INT4 MoE pipeline output against oracle.moe.forward on those tokens alone (a token's result
    depends on no other token).  `experts` may carry already dequantised (w13d, w2d) to share them between calls."""
    w13d, w2d = experts if experts is not None else (LazyExperts(w13_i32, s13, x.dtype), LazyExperts(w2_i32, s2, x.dtype))
    ref = moe.forward(_rows(x, toks), _rows(logits, toks), w13d, w2d, top_k, round_intermediates=True)
    return errors(_rows(out, toks), ref)
