"""All ten callables of the C++ extension, called the way upstream's autograd wrappers call
their compiled backend (src/ssm/ops/__init__.py:294-471, 570-676, 785-900, 961-1034, 1127-1224),
against the oracle's outputs and autograd gradients.

The case matrix (option combinations, shapes, fp32 and fp16 with B / C / D / dt_bias in the
activation dtype, ``sum()`` losses over output and state) is the one of upstream's backend-parity
tests (tests/ops/test_backend_gradients.py:24-46 and the case tables at :186-350); the fp16 bars are
upstream's (:134-147), the fp32 bars the tighter ones used everywhere else in this suite.
"""

from __future__ import annotations

import pytest
import torch

from oracle import ssm_oracle as orc
from tests.gpu_util import FP32_TOL, REDUCED, close

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16]


def _tol(dtype, grad=False):
    if dtype == torch.float16:
        return dict(rtol=5e-3, atol=5e-3) if grad else dict(rtol=3e-3, atol=2e-3)
    return FP32_TOL


def _ext():
    from ssm_b200 import backend

    return backend.load_extension()


def _mk(gen, *shape, dtype=torch.float32, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(dtype)


def _check_grads(names, got, want, dtype, tag):
    for k, a, b in zip(names, got, want):
        if b is None:
            assert a is None, f"{tag}: unexpected gradient for {k}"
            continue
        assert a is not None, f"{tag}: no gradient for {k}"
        assert a.dtype == b.dtype and a.shape == b.shape, f"{tag} d{k}: {a.dtype} {tuple(a.shape)} vs {b.dtype} {tuple(b.shape)}"
        close(a, b, **_tol(dtype, grad=True), what=f"{tag} d{k}", reduced=k in REDUCED)


SCAN_CASES = [
    dict(name="full", return_last_state=True, softplus=True, with_D=True, with_z=True, with_dt_bias=True),
    dict(name="minimal", return_last_state=False, softplus=False, with_D=False, with_z=False, with_dt_bias=False),
    dict(name="partial", return_last_state=True, softplus=False, with_D=True, with_z=False, with_dt_bias=True),
    dict(name="gate_only", return_last_state=False, softplus=True, with_D=False, with_z=True, with_dt_bias=False),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "f16"])
@pytest.mark.parametrize("case", SCAN_CASES, ids=[c["name"] for c in SCAN_CASES])
@pytest.mark.parametrize("shape", [(2, 3, 4, 5), (2, 48, 16, 150)], ids=["upstream-shape", "wide"])
def test_selective_scan_and_backward(case, dtype, shape):
    ext = _ext()
    gen = torch.Generator().manual_seed(101)
    nb, nd, nn, nl = shape
    delta = _mk(gen, nb, nd, nl, dtype=dtype, scale=0.5)
    if not case["softplus"] and nl > 16:
        delta = delta.abs() + 1.5  # a raw negative step (after the bias) makes the recurrence grow without bound over a long sequence
    ins = dict(u=_mk(gen, nb, nd, nl, dtype=dtype), delta=delta, A=-torch.exp(_mk(gen, nd, nn, scale=0.5)),
               B=_mk(gen, nd, nn, dtype=dtype), C=_mk(gen, nd, nn, dtype=dtype),
               D=_mk(gen, nd, dtype=dtype) if case["with_D"] else None, z=_mk(gen, nb, nd, nl, dtype=dtype) if case["with_z"] else None,
               dt_bias=_mk(gen, nd, dtype=dtype, scale=0.5) if case["with_dt_bias"] else None)
    lo = {k: (None if v is None else v.clone().requires_grad_(True)) for k, v in ins.items()}
    g = {k: (None if v is None else v.cuda()) for k, v in ins.items()}
    want = orc.selective_scan(lo["u"], lo["delta"], lo["A"], lo["B"], lo["C"], D=lo["D"], z=lo["z"], dt_bias=lo["dt_bias"],
                              softplus=case["softplus"], return_last_state=case["return_last_state"])
    yo, so = want if case["return_last_state"] else (want, None)
    out, last, cache = ext.selective_scan(g["u"], g["delta"], g["A"], g["B"], g["C"], g["D"], g["z"], g["dt_bias"], case["softplus"],
                                          case["return_last_state"])
    assert out.dtype == dtype and cache.dtype == torch.float32
    close(out, yo, **_tol(dtype), what="out")
    if so is None:
        assert last.numel() == 0
    else:
        assert last.dtype == dtype
        close(last, so, **_tol(dtype), what="last_state")
    loss = yo.float().sum() + (0 if so is None else so.float().sum())
    live = [k for k, v in lo.items() if v is not None]
    go = dict(zip(live, torch.autograd.grad(loss, [lo[k] for k in live])))
    grads = ext.selective_scan_backward(torch.ones_like(out), None if so is None else torch.ones_like(last), g["u"], g["delta"], g["A"], g["B"], g["C"],
                                        g["D"], g["z"], g["dt_bias"], case["softplus"], out, cache)
    assert len(grads) == 8
    names = ["u", "delta", "A", "B", "C", "D", "z", "dt_bias"]
    _check_grads(names, grads, [go.get(k) for k in names], dtype, f"scan/{case['name']}")
    # without a cache the backward produces the checkpoints itself
    again = ext.selective_scan_backward(torch.ones_like(out), None if so is None else torch.ones_like(last), g["u"], g["delta"], g["A"], g["B"], g["C"],
                                        g["D"], g["z"], g["dt_bias"], case["softplus"], out, torch.empty(0, device="cuda"))
    assert torch.equal(again[0], grads[0])


def test_selective_scan_grouped_time_varying_coefficients_through_the_extension():
    ext = _ext()
    gen = torch.Generator().manual_seed(7)
    nb, nd, nn, nl = 2, 32, 16, 96
    ins = dict(u=_mk(gen, nb, nd, nl), delta=_mk(gen, nb, nd, nl, scale=0.5), A=-torch.exp(_mk(gen, nd, nn, scale=0.5)), B=_mk(gen, nb, 2, nn, nl),
               C=_mk(gen, nb, 1, nn, nl))
    lo = {k: v.clone().requires_grad_(True) for k, v in ins.items()}
    g = {k: v.cuda() for k, v in ins.items()}
    yo, so = orc.selective_scan(lo["u"], lo["delta"], lo["A"], lo["B"], lo["C"], softplus=True, return_last_state=True)
    out, last, cache = ext.selective_scan(g["u"], g["delta"], g["A"], g["B"], g["C"], None, None, None, True, True)
    close(out, yo, **FP32_TOL, what="out")
    close(last, so, **FP32_TOL, what="last")
    go = torch.autograd.grad(yo.sum() + so.sum(), list(lo.values()))
    grads = ext.selective_scan_backward(torch.ones_like(out), torch.ones_like(last), g["u"], g["delta"], g["A"], g["B"], g["C"], None, None, None, True,
                                        out, cache)
    _check_grads(list(ins), grads[:5], go, torch.float32, "scan/grouped")  # dC comes back in C's one-group shape


STEP_CASES = [
    dict(name="full", softplus=True, with_D=True, with_z=True, with_dt_bias=True),
    dict(name="minimal", softplus=False, with_D=False, with_z=False, with_dt_bias=False),
    dict(name="skip_z", softplus=True, with_D=True, with_z=False, with_dt_bias=True),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "f16"])
@pytest.mark.parametrize("case", STEP_CASES, ids=[c["name"] for c in STEP_CASES])
@pytest.mark.parametrize("grouped", [False, True], ids=["per-channel", "grouped"])
def test_selective_state_step_and_backward(case, dtype, grouped):
    ext = _ext()
    gen = torch.Generator().manual_seed(102)
    nb, nd, nn = (2, 3, 4) if not grouped else (3, 24, 16)
    shp = (nd, nn) if not grouped else (nb, 2, nn)
    ins = dict(state=_mk(gen, nb, nd, nn, dtype=dtype, scale=0.3), x=_mk(gen, nb, nd, dtype=dtype), dt=_mk(gen, nb, nd, dtype=dtype, scale=0.5),
               A=-torch.exp(_mk(gen, nd, nn, scale=0.5)), B=_mk(gen, *shp, dtype=dtype), C=_mk(gen, *shp, dtype=dtype),
               D=_mk(gen, nd, dtype=dtype) if case["with_D"] else None, z=_mk(gen, nb, nd, dtype=dtype) if case["with_z"] else None,
               dt_bias=_mk(gen, nd, dtype=dtype, scale=0.5) if case["with_dt_bias"] else None)
    lo = {k: (None if v is None else v.clone().requires_grad_(True)) for k, v in ins.items()}
    g = {k: (None if v is None else v.cuda()) for k, v in ins.items()}
    yo, no = orc.selective_state_step(lo["state"], lo["x"], lo["dt"], lo["A"], lo["B"], lo["C"], D=lo["D"], z=lo["z"], dt_bias=lo["dt_bias"],
                                      softplus=case["softplus"], inplace=False)
    work = g["state"].clone()
    y = ext.selective_state_step(work, g["x"], g["dt"], g["A"], g["B"], g["C"], g["D"], g["z"], g["dt_bias"], case["softplus"])
    assert y.dtype == dtype and work.dtype == dtype
    close(y, yo, **_tol(dtype), what="y")
    close(work, no, **_tol(dtype), what="state (updated in place)")
    live = [k for k, v in lo.items() if v is not None]
    go = dict(zip(live, torch.autograd.grad(yo.float().sum() + no.float().sum(), [lo[k] for k in live])))
    grads = ext.selective_state_step_backward(torch.ones_like(y), torch.ones_like(work), g["state"], g["x"], g["dt"], g["A"], g["B"], g["C"], g["D"],
                                              g["z"], g["dt_bias"], case["softplus"])
    assert len(grads) == 9  # upstream's wrapper zips them with its nine requires_grad flags
    names = ["state", "x", "dt", "A", "B", "C", "D", "z", "dt_bias"]
    _check_grads(names, grads, [go.get(k) for k in names], dtype, f"step/{case['name']}")


CHUNK_CASES = [
    dict(name="full", with_D=True, with_z=True, with_seq_meta=True, with_initial_state=True),
    dict(name="minimal", with_D=False, with_z=False, with_seq_meta=False, with_initial_state=False),
    dict(name="ragged", with_D=False, with_z=True, with_seq_meta=True, with_initial_state=False),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "f16"])
@pytest.mark.parametrize("case", CHUNK_CASES, ids=[c["name"] for c in CHUNK_CASES])
@pytest.mark.parametrize("shape", [(2, 4, 3, 2, 2), (2, 75, 3, 16, 32)], ids=["upstream-shape", "longer"])
def test_ssd_chunk_scan_and_backward(case, dtype, shape):
    ext = _ext()
    gen = torch.Generator().manual_seed(103)
    nb, nl, nh, npj, chunk = shape
    zshape = (nb, nl, nh, npj) if case["name"] == "ragged" else (nb, nl, nh)
    ins = dict(X=_mk(gen, nb, nl, nh, npj, dtype=dtype), dt=(torch.rand(nb, nl, nh, generator=gen) * 0.5).to(dtype), A=-torch.exp(_mk(gen, nh, npj, scale=0.5)),
               B=_mk(gen, *(zshape if len(zshape) == 4 else (nh, npj)), dtype=dtype), C=_mk(gen, *(zshape if len(zshape) == 4 else (nh, npj)), dtype=dtype),
               D=_mk(gen, nh, dtype=dtype) if case["with_D"] else None,
               z=_mk(gen, *zshape, dtype=dtype) if case["with_z"] else None,
               initial_states=_mk(gen, nb, nh, npj, dtype=dtype) if case["with_initial_state"] else None)
    lens = torch.tensor([nl, nl - 1], dtype=torch.int64) if case["with_seq_meta"] else None
    lo = {k: (None if v is None else v.clone().requires_grad_(True)) for k, v in ins.items()}
    g = {k: (None if v is None else v.cuda()) for k, v in ins.items()}
    Yo = orc.ssd_chunk_scan(lo["X"], lo["dt"], lo["A"], lo["B"], lo["C"], chunk, D=lo["D"], z=lo["z"],
                            seq_meta=None if lens is None else {"seq_lens": lens}, initial_states=lo["initial_states"])
    glens = None if lens is None else lens.cuda()
    Y = ext.ssd_chunk_scan(g["X"], g["dt"], g["A"], g["B"], g["C"], chunk, g["D"], g["z"], glens, None, g["initial_states"])
    close(Y, Yo, **_tol(dtype), what="Y")
    if lens is not None:  # the cumulative form of the same lengths
        cu = torch.tensor([0, nl, 2 * nl - 1], dtype=torch.int64).cuda()
        assert torch.equal(ext.ssd_chunk_scan(g["X"], g["dt"], g["A"], g["B"], g["C"], chunk, g["D"], g["z"], None, cu, g["initial_states"]), Y)
    live = [k for k, v in lo.items() if v is not None]
    go = dict(zip(live, torch.autograd.grad(Yo.float().sum(), [lo[k] for k in live], allow_unused=True)))
    grads = ext.ssd_chunk_scan_backward(torch.ones_like(Y), g["X"], g["dt"], g["A"], g["B"], g["C"], chunk, g["D"], g["z"], glens, None,
                                        g["initial_states"])
    assert len(grads) == 8
    names = ["X", "dt", "A", "B", "C", "D", "z", "initial_states"]
    _check_grads(names, grads, [go.get(k) for k in names], dtype, f"chunk/{case['name']}")


CONV_CASES = [dict(name="identity_bias", with_bias=True, activation="identity"), dict(name="silu_no_bias", with_bias=False, activation="silu")]


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "f16"])
@pytest.mark.parametrize("case", CONV_CASES, ids=[c["name"] for c in CONV_CASES])
@pytest.mark.parametrize("first", [True, False], ids=["channels-first", "channels-last"])
def test_dw_causal_conv_and_backward(case, dtype, first):
    ext = _ext()
    gen = torch.Generator().manual_seed(104)
    nb, nc, nl, k = 2, 6, 37, 3
    x = _mk(gen, *((nb, nc, nl) if first else (nb, nl, nc)), dtype=dtype)
    w = _mk(gen, nc, 1, k, dtype=dtype, scale=0.5)  # upstream's modules store (C, 1, K)
    b = _mk(gen, nc, dtype=dtype) if case["with_bias"] else None
    lo = [t if t is None else t.clone().requires_grad_(True) for t in (x, w, b)]
    yo = orc.dw_causal_conv(lo[0], lo[1], lo[2], case["activation"])
    y = ext.dw_causal_conv(x.cuda(), w.cuda(), None if b is None else b.cuda(), case["activation"])
    close(y, yo, **_tol(dtype), what="y")
    go = torch.autograd.grad(yo.float().sum(), [t for t in lo if t is not None])
    dx, dw, db = ext.dw_causal_conv_backward(torch.ones_like(y), x.cuda(), w.cuda(), None if b is None else b.cuda(), case["activation"])
    _check_grads(["x", "weight", "bias"], [dx, dw, db], list(go) + ([None] if b is None else []), dtype, f"conv/{case['name']}")


NORM_CASES = [
    dict(name="prenorm_full", with_bias=True, with_residual=True, is_rms=False, prenorm=True, residual_in_fp32=True),
    dict(name="postnorm_rms", with_bias=False, with_residual=True, is_rms=True, prenorm=False, residual_in_fp32=False),
    dict(name="no_residual", with_bias=True, with_residual=False, is_rms=False, prenorm=False, residual_in_fp32=True),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "f16"])
@pytest.mark.parametrize("case", NORM_CASES, ids=[c["name"] for c in NORM_CASES])
@pytest.mark.parametrize("hidden", [6, 768], ids=["upstream-shape", "hidden768"])
def test_fused_layer_norm_and_backward(case, dtype, hidden):
    ext = _ext()
    gen = torch.Generator().manual_seed(105)
    x, w = _mk(gen, 2, 5, hidden, dtype=dtype), _mk(gen, hidden, dtype=dtype)
    b = _mk(gen, hidden, dtype=dtype) if case["with_bias"] else None
    res = _mk(gen, 2, 5, hidden, dtype=dtype) if case["with_residual"] else None
    lo = [t if t is None else t.clone().requires_grad_(True) for t in (x, w, b, res)]
    kw = dict(is_rms=case["is_rms"], eps=1e-5, prenorm=case["prenorm"], residual_in_fp32=case["residual_in_fp32"])
    yo = orc.fused_layer_norm(lo[0], lo[1], lo[2], residual=lo[3], **kw)
    c = lambda t: None if t is None else t.cuda()  # noqa: E731
    y = ext.fused_layer_norm(c(x), c(w), c(b), c(res), **kw)
    assert y.dtype == dtype
    close(y, yo, **_tol(dtype), what="y")
    go = iter(torch.autograd.grad(yo.float().sum(), [t for t in lo if t is not None]))
    want = [next(go) if t is not None else None for t in lo]
    grads = ext.fused_layer_norm_backward(torch.ones_like(y), c(x), c(w), c(b), c(res), **kw)
    assert len(grads) == 4
    for name, got, exp in zip(("x", "weight", "bias", "residual"), grads, want):
        if exp is None:
            assert got.numel() == 0, f"absent {name} must come back as an empty tensor"
        else:
            close(got, exp, **_tol(dtype, grad=True), what=f"norm/{case['name']} d{name}", reduced=name in REDUCED)


def test_backend_object_adapts_selective_scan_to_both_upstream_call_sites():
    """Upstream's autograd wrapper unpacks three values, its no-grad path two (src/ssm/ops/__init__.py:317, 1304)."""
    from ssm_b200.backend import Backend

    be = Backend()
    u, delta = torch.randn(1, 4, 9, device="cuda"), torch.rand(1, 4, 9, device="cuda")
    A, Bm, Cm = -torch.rand(4, 2, device="cuda"), torch.randn(4, 2, device="cuda"), torch.randn(4, 2, device="cuda")
    out, last = be.selective_scan(u, delta, A, Bm, Cm)
    assert last.numel() == 0 and out.shape == u.shape
    out3 = be.selective_scan(u.requires_grad_(True), delta, A, Bm, Cm, return_last_state=True)
    assert len(out3) == 3 and out3[1].shape == (1, 4, 2) and out3[2].dtype == torch.float32
    with pytest.raises(RuntimeError, match="delta must match"):
        be.selective_scan(u, delta[..., :8], A, Bm, Cm)
