"""Helpers shared by the GPU parity tests.

Comparison bars.  Element-wise tensors (outputs, final states, gradients that have the shape
of an activation) are held to the stated bars as they are: fp32 ``rtol 1e-4 / atol 1e-5``;
bf16 / fp16 I/O ``rtol 2e-2`` against the fp32 computation on the same rounded inputs, with a
small absolute term for values that cancel to nearly zero.  Only contractions over thousands
of terms -- parameter gradients summed over batch and time (``dA, dB, dC, dD, ddt_bias``, conv
and norm ``dweight / dbias``) and the outputs of the tensor-core SSD path, each a 256-term
bf16 product sum -- get the absolute term scaled by the magnitude of the expected tensor
(``reduced=True``): their rounding error grows with the size of the terms, not of the result.

The dual-form (tensor-core) backward of the SSD scan adds one more kind: gradients that sum
terms of both signs over batch and time (``dA``, ``ddt_bias``) out of 16-bit-operand
contractions.  Each term carries about 0.3 % of its own size, so the sum is held to a fraction
of the sum of the terms' magnitudes (``close_sum``), which is what conditions it -- the result
itself may cancel to far less.
"""

from __future__ import annotations

import torch

FP32_TOL = dict(rtol=1e-4, atol=1e-5)  # fp32 bar for outputs, final states and gradients
HALF_TOL = dict(rtol=2e-2, atol=2e-3)  # bf16 / fp16 I/O against the fp32 computation

# names of operator arguments whose gradient is a sum over batch and / or time
REDUCED = frozenset({"A", "B", "C", "D", "dt_bias", "weight", "bias", "A_log"})


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


def close(got, want, rtol, atol, what="", reduced=False):
    """``|got - want| <= atol + rtol * |want|`` element by element.  ``reduced=True`` scales the
    absolute term by ``max(1, max|want|)`` (contractions over many terms; see the module text)."""
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    ok = torch.isfinite(want)
    scale = 1.0
    if reduced and ok.any():
        scale = max(1.0, float(want[ok].abs().max()))
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


def close_sum(got, want, abs_terms, frac, what=""):
    """``|got - want| <= frac * abs_terms`` element by element: for a sum of signed terms, ``abs_terms`` being (an estimate
    of) the sum of their magnitudes."""
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    abs_terms = abs_terms.detach().float().cpu()
    assert got.shape == want.shape == abs_terms.shape, f"{what}: shapes {tuple(got.shape)}, {tuple(want.shape)}, {tuple(abs_terms.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - want).abs()
    bad = err > frac * abs_terms
    if bad.any():
        i = int(torch.argmax(err / abs_terms.clamp_min(1e-30)))
        raise AssertionError(f"{what}: {int(bad.sum())}/{bad.numel()} off; worst |err|={float(err.flatten()[i]):.3e} "
                             f"(got {float(got.flatten()[i]):.6e}, want {float(want.flatten()[i]):.6e}, sum of |terms| {float(abs_terms.flatten()[i]):.3e})")
