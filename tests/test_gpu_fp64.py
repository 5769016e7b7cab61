"""float64 variants of the five operators: values against the oracle in float64 and ``torch.autograd.gradcheck`` (what upstream
runs on its CUDA backend, tests/ops/test_backend_gradients.py:1172-1612)."""

from __future__ import annotations

import pytest
import torch

from oracle import ssm_oracle as orc

pytestmark = pytest.mark.gpu

DD = torch.float64


def _r(gen, *shape, scale=1.0, grad=True):
    return (torch.randn(*shape, generator=gen, dtype=DD) * scale).cuda().requires_grad_(grad)


def _check(fn, inputs):
    assert torch.autograd.gradcheck(fn, inputs, eps=1e-6, atol=1e-6, rtol=1e-5, nondet_tol=1e-9)


@pytest.mark.parametrize("layout", ["shared", "per_batch", "grouped_time"])
def test_selective_scan(layout):
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(1)
    nb, nd, nl, nn = 2, 4, 7, 3
    u, delta, z = _r(gen, nb, nd, nl), _r(gen, nb, nd, nl, scale=0.5), _r(gen, nb, nd, nl)
    A = (-torch.exp(torch.randn(nd, nn, generator=gen, dtype=DD) * 0.3)).cuda().requires_grad_(True)
    shape = {"shared": (nd, nn), "per_batch": (nb, nd, nn), "grouped_time": (nb, 2, nn, nl)}[layout]
    Bm, Cm = _r(gen, *shape), _r(gen, *shape)
    D, bias, init = _r(gen, nd), _r(gen, nd, scale=0.3), _r(gen, nb, nd, nn, scale=0.5)

    def fn(u, delta, A, Bm, Cm, D, z, bias, init):
        return ops.selective_scan(u, delta, A, Bm, Cm, D=D, z=z, dt_bias=bias, softplus=True, return_last_state=True, initial_state=init)

    y, last = fn(u, delta, A, Bm, Cm, D, z, bias, init)
    c = [t.detach().cpu() for t in (u, delta, A, Bm, Cm, D, z, bias, init)]
    yo, lo = orc.selective_scan(c[0], c[1], c[2], c[3], c[4], D=c[5], z=c[6], dt_bias=c[7], softplus=True, return_last_state=True,
                                initial_state=c[8])
    torch.testing.assert_close(y.cpu(), yo, rtol=1e-10, atol=1e-10)
    torch.testing.assert_close(last.cpu(), lo.to(DD), rtol=1e-10, atol=1e-10)
    _check(fn, (u, delta, A, Bm, Cm, D, z, bias, init))


@pytest.mark.parametrize("grouped", [False, True])
def test_selective_state_step(grouped):
    from ssm_b200 import ops_f64

    gen = torch.Generator().manual_seed(2)
    nb, nd, nn = 3, 4, 5
    state, x, dt, z = _r(gen, nb, nd, nn), _r(gen, nb, nd), _r(gen, nb, nd, scale=0.5), _r(gen, nb, nd)
    A = (-torch.exp(torch.randn(nd, nn, generator=gen, dtype=DD) * 0.3)).cuda().requires_grad_(True)
    Bm, Cm = (_r(gen, nb, 2, nn), _r(gen, nb, 2, nn)) if grouped else (_r(gen, nd, nn), _r(gen, nd, nn))
    D, bias = _r(gen, nd), _r(gen, nd, scale=0.3)

    def fn(state, x, dt, A, Bm, Cm, D, z, bias):
        return ops_f64.selective_state_step_functional(state, x, dt, A, Bm, Cm, D=D, z=z, dt_bias=bias, softplus=True)

    y, new = fn(state, x, dt, A, Bm, Cm, D, z, bias)
    so = state.detach().cpu().clone()
    yo = orc.selective_state_step(so, x.detach().cpu(), dt.detach().cpu(), A.detach().cpu(), Bm.detach().cpu(), Cm.detach().cpu(),
                                  D=D.detach().cpu(), z=z.detach().cpu(), dt_bias=bias.detach().cpu(), softplus=True)
    torch.testing.assert_close(y.cpu(), yo, rtol=1e-10, atol=1e-10)
    torch.testing.assert_close(new.cpu(), so, rtol=1e-10, atol=1e-10)
    _check(fn, (state, x, dt, A, Bm, Cm, D, z, bias))


def test_selective_state_step_in_place():
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(3)
    nb, nd, nn = 2, 3, 4
    state = _r(gen, nb, nd, nn, grad=False)
    x, dt = _r(gen, nb, nd, grad=False), _r(gen, nb, nd, scale=0.5, grad=False)
    A = (-torch.exp(torch.randn(nd, nn, generator=gen, dtype=DD) * 0.3)).cuda()
    Bm, Cm = _r(gen, nd, nn, grad=False), _r(gen, nd, nn, grad=False)
    so = state.cpu().clone()
    y = ops.selective_state_step(state, x, dt, A, Bm, Cm, softplus=True)
    yo = orc.selective_state_step(so, x.cpu(), dt.cpu(), A.cpu(), Bm.cpu(), Cm.cpu(), softplus=True)
    torch.testing.assert_close(y.cpu(), yo, rtol=1e-10, atol=1e-10)
    torch.testing.assert_close(state.cpu(), so, rtol=1e-10, atol=1e-10)


@pytest.mark.parametrize("kind", ["shared", "time_varying"])
def test_ssd_chunk_scan(kind):
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(4)
    nb, nl, nh, npj = 2, 6, 2, 3
    X, dt = _r(gen, nb, nl, nh, npj), (torch.rand(nb, nl, nh, generator=gen, dtype=DD) * 0.5 + 0.1).cuda().requires_grad_(True)
    A = (-torch.rand(nh, npj, generator=gen, dtype=DD) - 0.2).cuda().requires_grad_(True)
    if kind == "shared":
        Bm, Cm, z, D = _r(gen, nh, npj), _r(gen, nh, npj), _r(gen, nb, nl, nh), _r(gen, nh)
    else:
        Bm, Cm, z, D = _r(gen, nb, nl, nh, npj), _r(gen, nb, nl, nh, npj), _r(gen, nb, nl, nh, npj), _r(gen, nh, npj)
    init = _r(gen, nb, nh, npj)
    meta = {"seq_lens": torch.tensor([nl, nl - 2])}

    def fn(X, dt, A, Bm, Cm, D, z, init):
        return ops.ssd_chunk_scan(X, dt, A, Bm, Cm, 4, D=D, z=z, seq_meta=meta, initial_states=init)

    Y = fn(X, dt, A, Bm, Cm, D, z, init)
    c = [t.detach().cpu() for t in (X, dt, A, Bm, Cm, D, z, init)]
    Yo = orc.ssd_chunk_scan(c[0], c[1], c[2], c[3], c[4], 4, D=c[5], z=c[6], seq_meta=meta, initial_states=c[7])
    torch.testing.assert_close(Y.cpu(), Yo, rtol=1e-10, atol=1e-10)
    _check(fn, (X, dt, A, Bm, Cm, D, z, init))


@pytest.mark.parametrize("first,act", [(True, "silu"), (False, "identity")])
def test_dw_causal_conv(first, act):
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(5)
    nb, nc, nl, k = 2, 3, 6, 4
    x = _r(gen, nb, nc, nl) if first else _r(gen, nb, nl, nc)
    w, b = _r(gen, nc, k, scale=0.5), _r(gen, nc, scale=0.3)

    def fn(x, w, b):
        return ops.dw_causal_conv(x, w, b, act)

    y = fn(x, w, b)
    yo = orc.dw_causal_conv(x.detach().cpu(), w.detach().cpu(), b.detach().cpu(), act)
    torch.testing.assert_close(y.cpu(), yo, rtol=1e-10, atol=1e-10)
    _check(fn, (x, w, b))


@pytest.mark.parametrize("is_rms,prenorm,with_res", [(True, True, True), (False, True, True), (False, False, True), (True, True, False)])
def test_fused_layer_norm(is_rms, prenorm, with_res):
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(6)
    nb, nl, nd = 2, 3, 5
    x, w, b = _r(gen, nb, nl, nd), _r(gen, nd), _r(gen, nd, scale=0.3)
    res = _r(gen, nb, nl, nd) if with_res else None

    def fn(x, w, b, *r):
        return ops.fused_layer_norm(x, w, b, r[0] if r else None, is_rms=is_rms, eps=1e-5, prenorm=prenorm, residual_in_fp32=False,
                                    return_residual=True)

    ins = (x, w, b, res) if with_res else (x, w, b)
    y, ro = fn(*ins)
    yo, roo = orc.fused_layer_norm(x.detach().cpu(), w.detach().cpu(), b.detach().cpu(), None if res is None else res.detach().cpu(),
                                   is_rms=is_rms, eps=1e-5, prenorm=prenorm, residual_in_fp32=False, return_residual=True)
    torch.testing.assert_close(y.cpu(), yo.to(DD), rtol=1e-10, atol=1e-10)
    torch.testing.assert_close(ro.cpu(), roo.to(DD), rtol=1e-10, atol=1e-10)
    _check(fn, ins)


def test_backend_entry_points_in_float64():
    """The installed backend serves upstream's ten names for float64 tensors too (forward values against the oracle, the
    backward tuples against autograd through the oracle)."""
    from ssm_b200.backend import Backend

    be = Backend()
    gen = torch.Generator().manual_seed(9)
    nb, nd, nl, nn = 2, 4, 5, 3
    mk = lambda *s, scale=1.0: (torch.randn(*s, generator=gen, dtype=DD) * scale)  # noqa: E731
    u, delta, z = mk(nb, nd, nl), mk(nb, nd, nl, scale=0.5), mk(nb, nd, nl)
    A, Bm, Cm = -torch.exp(mk(nd, nn, scale=0.3)), mk(nb, 2, nn, nl), mk(nb, 2, nn, nl)
    D, bias = mk(nd), mk(nd, scale=0.3)
    cpu = [u, delta, A, Bm, Cm, D, z, bias]
    leaves = [t.clone().requires_grad_(True) for t in cpu]
    yo, lo = orc.selective_scan(*leaves[:5], D=leaves[5], z=leaves[6], dt_bias=leaves[7], softplus=True, return_last_state=True)
    gy, gl = mk(nb, nd, nl), mk(nb, nd, nn)
    want = torch.autograd.grad((yo * gy).sum() + (lo * gl).sum(), leaves)
    dev = [t.cuda() for t in cpu]
    out, last = be.selective_scan(*dev[:5], D=dev[5], z=dev[6], dt_bias=dev[7], softplus=True, return_last_state=True)
    torch.testing.assert_close(out.cpu(), yo.detach(), rtol=1e-10, atol=1e-10)
    torch.testing.assert_close(last.cpu(), lo.detach().to(DD), rtol=1e-10, atol=1e-10)
    got = be.selective_scan_backward(gy.cuda(), gl.cuda(), *dev[:5], dev[5], dev[6], dev[7], True, out, out.new_empty(0))
    assert len(got) == 8
    for g, w in zip(got, want):
        torch.testing.assert_close(g.cpu(), w, rtol=1e-9, atol=1e-9)
    # conv and norm: arities of the backward tuples
    x, w, b = mk(nb, nd, nl).cuda(), mk(nd, 4, scale=0.5).cuda(), mk(nd).cuda()
    y = be.dw_causal_conv(x, w, b, "silu")
    torch.testing.assert_close(y.cpu(), orc.dw_causal_conv(x.cpu(), w.cpu(), b.cpu(), "silu"), rtol=1e-10, atol=1e-10)
    assert len(be.dw_causal_conv_backward(torch.ones_like(y), x, w, b, "silu")) == 3
    xs, ws = mk(nb, nl, nd).cuda(), mk(nd).cuda()
    yn = be.fused_layer_norm(xs, ws, None, None, True, 1e-5, True, False)
    torch.testing.assert_close(yn.cpu(), orc.fused_layer_norm(xs.cpu(), ws.cpu(), None, None, is_rms=True, residual_in_fp32=False),
                               rtol=1e-10, atol=1e-10)
    assert len(be.fused_layer_norm_backward(torch.ones_like(yn), xs, ws, None, None, True, 1e-5, True, False)) == 4
    st = mk(nb, nd, nn).cuda()
    so = st.cpu().clone()
    xs2, dts = mk(nb, nd).cuda(), mk(nb, nd, scale=0.5).cuda()
    ys = be.selective_state_step(st, xs2, dts, A.cuda(), mk(nd, nn).cuda(), mk(nd, nn).cuda())
    assert ys.shape == (nb, nd) and not torch.equal(st.cpu(), so)
    assert len(be.selective_state_step_backward(torch.ones_like(ys), None, st, xs2, dts, A.cuda(), mk(nd, nn).cuda(), mk(nd, nn).cuda(),
                                                None, None, None, True)) == 9
    X, dt2 = mk(nb, nl, 2, 3).cuda(), (torch.rand(nb, nl, 2, generator=gen, dtype=DD) * 0.5).cuda()
    A2, B2, C2 = -torch.rand(2, 3, generator=gen, dtype=DD).cuda(), mk(2, 3).cuda(), mk(2, 3).cuda()
    Y = be.ssd_chunk_scan(X, dt2, A2, B2, C2, 4)
    torch.testing.assert_close(Y.cpu(), orc.ssd_chunk_scan(X.cpu(), dt2.cpu(), A2.cpu(), B2.cpu(), C2.cpu(), 4), rtol=1e-10, atol=1e-10)
    assert len(be.ssd_chunk_scan_backward(torch.ones_like(Y), X, dt2, A2, B2, C2, 4, None, None, None, None, None)) == 8
