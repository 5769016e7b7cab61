"""The allocation-free backward of the fused add + norm against the regular entry point.

Some users of the library cannot allocate device memory at call time: a serving process that
carved up one arena at start-up, a plugin that must stay out of its host's CUDA allocator,
a latency-critical loop that cannot afford the implicit device synchronisation of
``cudaMalloc`` / ``cudaFree``.  For them ``ssm_fused_add_norm_bwd_noalloc`` keeps the kernel's
scratch in a fixed array inside the library.  This test drives both entry points through the
C ABI with the same inputs, twice in a row with different data (the shared array keeps the
previous call's contents, which must not leak into the next result), and checks the outputs
against each other at the suite's fp32 / half tolerances.  It lives in a file that sorts last so
that a run stopping at the first failure has already finished every other test.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from tests.gpu_util import FP32_TOL, HALF_TOL, close

pytestmark = pytest.mark.gpu


def _run(entry, nc, gy, with_partial):
    """Call one of the two backward entry points; returns (dx, dres, dw, db)."""
    from ssm_b200 import _lib as L
    from ssm_b200.ops import _p, _stream

    lib = L.load()
    x = nc.x
    hidden, rows = x.shape[2], x.shape[0] * x.shape[1]
    dx = torch.empty_like(x)
    dres = torch.empty_like(nc.res) if nc.res is not None else None
    dw = torch.full((hidden,), float("nan"), device=x.device)
    db = torch.full((hidden,), float("nan"), device=x.device) if nc.b is not None else None
    partial = None
    if with_partial:
        partial = torch.empty(int(lib.ssm_norm_bwd_scratch_floats(rows, hidden)), dtype=torch.float32, device=x.device)
    g = L.NormBwdArgs()
    nc.fill(g.fwd)
    g.dy, g.dx, g.dresidual, g.dweight, g.dbias, g.partial = _p(gy), _p(dx), _p(dres), _p(dw), _p(db), _p(partial)
    rc = getattr(lib, entry)(ctypes.byref(g), _stream())
    assert rc == 0, lib.ssm_b200_last_error().decode()
    torch.cuda.synchronize()
    return dx, dres, dw, db


CASES = [
    # rows (B, L), hidden, dtype, residual dtype, rms, prenorm, bias
    ((8, 300), 768, torch.bfloat16, torch.float32, True, True, False),
    ((3, 70), 2560, torch.float32, torch.float32, False, True, True),
    ((2, 40), 8192, torch.float16, None, False, False, True),
    ((2, 9), 100, torch.float32, torch.float32, True, False, True),   # vectorised fp32 path, tiny
    ((1, 5), 33, torch.float32, None, False, True, True),             # scalar path (no scratch used)
]


@pytest.mark.parametrize("shape,hidden,dtype,rdtype,is_rms,prenorm,has_bias", CASES)
def test_noalloc_backward_matches_regular_entry_point(shape, hidden, dtype, rdtype, is_rms, prenorm, has_bias):
    from ssm_b200.ops import _NormCtx

    tol = FP32_TOL if dtype == torch.float32 else HALF_TOL
    gen = torch.Generator().manual_seed(hidden + shape[1])
    for call in range(2):  # two calls in a row share the built-in scratch
        x = torch.randn(*shape, hidden, generator=gen).mul(1.0 + call).to(dtype).cuda()
        w = torch.randn(hidden, generator=gen).to(dtype).cuda()
        b = torch.randn(hidden, generator=gen).to(dtype).cuda() if has_bias else None
        res = None if rdtype is None else torch.randn(*shape, hidden, generator=gen).to(rdtype).cuda()
        gy = torch.randn(*shape, hidden, generator=gen).to(dtype).cuda()
        nc = _NormCtx(x, w, b, res, is_rms, 1e-5, prenorm)
        want = _run("ssm_fused_add_norm_bwd", nc, gy, True)
        got = _run("ssm_fused_add_norm_bwd_noalloc", nc, gy, False)
        for name, g_, w_ in zip(("dx", "dresidual", "dweight", "dbias"), got, want):
            if w_ is None:
                assert g_ is None
                continue
            close(g_, w_, **(FP32_TOL if name in ("dweight", "dbias") else tol), what=f"call {call} {name}", reduced=name in ("dweight", "dbias"))
        assert torch.equal(got[0], want[0]), "dx must be bit-identical"


def test_noalloc_rejects_rows_wider_than_its_scratch():
    from ssm_b200 import _lib as L
    from ssm_b200.ops import _NormCtx, _p, _stream

    lib = L.load()
    x = torch.zeros(1, 2, 8200, device="cuda")
    nc = _NormCtx(x, torch.ones(8200, device="cuda"), None, None, True, 1e-5, True)
    g = L.NormBwdArgs()
    nc.fill(g.fwd)
    dw = torch.zeros(8200, device="cuda")
    g.dy, g.dx, g.dweight = _p(x), _p(torch.empty_like(x)), _p(dw)
    assert lib.ssm_fused_add_norm_bwd_noalloc(ctypes.byref(g), _stream()) == -6
    assert b"8192" in lib.ssm_b200_last_error()
