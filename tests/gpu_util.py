"""Helpers shared by the GPU parity tests."""

from __future__ import annotations

import torch

FP32_TOL = dict(rtol=1e-4, atol=1e-5)  # fp32 bar for outputs, final states and gradients
HALF_TOL = dict(rtol=2e-2, atol=2e-2)  # bf16 / fp16 I/O against the fp32 computation


def dev(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        return t.cuda()
    return t


def leaf(t, grad=True):
    if t is None:
        return None
    t = t.detach().clone().cuda()
    if grad and t.is_floating_point():
        t.requires_grad_(True)
    return t


def close(got, want, rtol, atol, what=""):
    """allclose with the absolute term scaled by the magnitude of the expected tensor, so that
    reductions over thousands of terms are judged relative to their own scale."""
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    ok = torch.isfinite(want)
    scale = max(1.0, float(want[ok].abs().max())) if ok.any() else 1.0
    err = (got[ok] - want[ok]).abs()
    bound = atol * scale + rtol * want[ok].abs()
    bad = err > bound
    if bad.any():
        i = int(torch.argmax(err - bound))
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.numel()} elements off; worst |err|={float(err[i]):.3e} "
            f"(got {float(got[ok][i]):.6e}, want {float(want[ok][i]):.6e}, bound {float(bound[i]):.3e})"
        )
    assert torch.isfinite(got[ok]).all(), f"{what}: non-finite values"
