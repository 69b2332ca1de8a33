"""Helpers for the GPU parity tests.  Tolerances (bf16 inputs, fp32 accumulation):

  out, dq, dk, dv : elementwise |got - ref| <= 2e-2 + 1e-2 * |ref|  and  relative L2 <= 1e-2
  lse             : max abs <= 1e-3

The absolute part is the max-abs bound for O(1) values; the relative part is what one bf16 ulp
(2^-8 relative) of the stored result needs once values exceed ~2.
"""
import torch

ATOL, RTOL, REL_L2, LSE_TOL = 2e-2, 1e-2, 1e-2, 1e-3


def assert_close(name, got, ref, atol=ATOL, rtol=RTOL, rel_l2=REL_L2):
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    err = (got - ref).abs()
    bound = atol + rtol * ref.abs()
    worst = (err - bound).max().item()
    assert worst <= 0, f"{name}: max abs err {err.max().item():.4g} exceeds atol {atol} + rtol {rtol}*|ref| by {worst:.4g}"
    denom = ref.norm().item()
    if denom > 0:
        r = (got - ref).norm().item() / denom
        assert r <= rel_l2, f"{name}: relative L2 {r:.4g} > {rel_l2}"


def assert_lse_close(got, ref, tol=LSE_TOL):
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    both_inf = torch.isinf(got) & torch.isinf(ref) & (got == ref)
    err = torch.where(both_inf, torch.zeros_like(got), (got - ref).abs())
    assert err.max().item() <= tol, f"lse: max abs err {err.max().item():.4g} > {tol}"


def randn_bf16(*shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).bfloat16()
