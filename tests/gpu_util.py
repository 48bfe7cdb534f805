"""Helpers shared by the GPU parity tests."""
import torch

DEV = "cuda:0"


def rel_errors(out: torch.Tensor, ref: torch.Tensor):
    """(max|d| / max|ref|, max elementwise relative error with the denominator clamped at 1e-3 max|ref|,
    mean|d| / mean|ref|, cosine) -- the error forms the reference's own tests report."""
    o, r = out.detach().float().cpu(), ref.detach().float().cpu()
    d = (o - r).abs()
    mx = r.abs().max().clamp(min=1e-30)
    e_max = float(d.max() / mx)
    e_el = float((d / r.abs().clamp(min=1e-3 * float(mx))).max())
    e_mean = float(d.mean() / r.abs().mean().clamp(min=1e-30))
    cos = float(torch.nn.functional.cosine_similarity(o.flatten(), r.flatten(), dim=0))
    return e_max, e_el, e_mean, cos


def assert_close(out, ref, tol=1e-2, what=""):
    """Gate: max|d|/max|ref| <= tol (1e-2 for a bf16/fp16 output of an fp32 accumulation)."""
    ref16 = ref.float()
    e_max, e_el, e_mean, cos = rel_errors(out, ref16)
    assert e_max <= tol, f"{what}: max_abs_err/max_abs_ref={e_max:.3e} (elementwise {e_el:.3e}, mean {e_mean:.3e}, cos {cos:.6f})"
    assert e_mean <= tol and cos > 0.9999, f"{what}: mean_rel={e_mean:.3e} cos={cos:.6f}"
