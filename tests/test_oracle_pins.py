"""Pins the CPU oracle (oracle/ssm_oracle.py) to the upstream package: every
known-answer vector upstream ships for the five operators, and the outputs and
gradients recorded by running upstream's own Python operators."""

from __future__ import annotations

import pytest
import torch

from oracle import ssm_oracle as orc
from tests.fixtures import cases, tol

PACKS = ("upstream_kats", "reference_runs")


def _leaf(t):
    if t is None:
        return None
    t = t.clone()
    return t.requires_grad_(True) if t.is_floating_point() else t


def _close(got, want, **kw):
    torch.testing.assert_close(got.float(), want.float(), **kw)


def _check_grads(case, outs, weights, leaves):
    if not case.grads:
        return
    live = {k: v for k, v in leaves.items() if v is not None and k in case.grads}
    total = sum((o.float() * w.float()).sum() for o, w in zip(outs, weights))
    got = torch.autograd.grad(total, list(live.values()), allow_unused=True)
    for (k, _), g in zip(live.items(), got):
        want = case.grads[k]
        ok = torch.isfinite(want)  # mamba-ssm's recorded gradients hold NaNs where its kernel overflowed
        _close(g[ok], want[ok], **tol(case, grad=True))


def _all(family):
    return [pytest.param(c, id=f"{p}:{c.name}") for p in PACKS for c in cases(p, family)]


@pytest.mark.parametrize("case", _all("scan"))
def test_selective_scan(case):
    i = {k: _leaf(v) for k, v in case.ins.items()}
    y, last = orc.selective_scan(i["u"], i["delta"], i["A"], i["B"], i["C"], D=i.get("D"), z=i.get("z"),
                                 dt_bias=i.get("dt_bias"), softplus=case.opts["softplus"], return_last_state=True)
    _close(y, case.outs["out"], **tol(case))
    if "last_state" in case.outs:
        _close(last, case.outs["last_state"], **tol(case))
    wy = i.get("grad_out")
    ws = i.get("grad_last_state")
    if wy is None:  # mamba-ssm vectors: loss = y.sum()
        _check_grads(case, (y,), (torch.ones_like(y),), i)
    else:
        _check_grads(case, (y, last), (wy.detach(), ws.detach()), i)


@pytest.mark.parametrize("case", _all("step"))
def test_selective_state_step(case):
    i = {k: v.clone() for k, v in case.ins.items()}
    state = i["state"]
    y = orc.selective_state_step(state, i["x"], i["dt"], i["A"], i["B"], i["C"], D=i.get("D"), z=i.get("z"),
                                 dt_bias=i.get("dt_bias"), softplus=case.opts["softplus"])
    _close(y, case.outs["y"], **tol(case))
    _close(state, case.outs["state"], **tol(case))


@pytest.mark.parametrize("case", _all("chunk"))
def test_ssd_chunk_scan(case):
    i = {k: _leaf(v) for k, v in case.ins.items()}
    meta = None
    if "cu_seqlens" in i:
        meta = {"cu_seqlens": i["cu_seqlens"]}
    elif "seq_lens" in i:
        meta = {"seq_lens": i["seq_lens"]}
    Y = orc.ssd_chunk_scan(i["X"], i["dt"], i["A"], i["B"], i["C"], case.opts["chunk_size"], D=i.get("D"), z=i.get("z"),
                           seq_meta=meta, initial_states=i.get("initial_states"))
    _close(Y, case.outs["Y"], **tol(case))
    if "grad_out" in i:
        _check_grads(case, (Y,), (i["grad_out"].detach(),), i)


@pytest.mark.parametrize("case", _all("conv"))
def test_dw_causal_conv(case):
    i = {k: _leaf(v) for k, v in case.ins.items()}
    y = orc.dw_causal_conv(i["x"], i["weight"], bias=i.get("bias"), activation=case.opts["activation"])
    _close(y, case.outs["y"], **tol(case))
    w = i["grad_out"].detach() if "grad_out" in i else torch.ones_like(y)
    _check_grads(case, (y,), (w,), i)


@pytest.mark.parametrize("case", _all("norm"))
def test_fused_layer_norm(case):
    i = {k: _leaf(v) for k, v in case.ins.items()}
    o = case.opts
    y, res = orc.fused_layer_norm(i["x"], i["weight"], i.get("bias"), residual=i.get("residual"), is_rms=o["is_rms"],
                                  eps=o["eps"], prenorm=o["prenorm"], residual_in_fp32=o.get("residual_in_fp32", True),
                                  return_residual=True)
    _close(y, case.outs["y"], **tol(case))
    if "residual_out" in case.outs:
        _close(res, case.outs["residual_out"], **tol(case))
    w = i["grad_out"].detach() if "grad_out" in i else torch.ones_like(y)
    _check_grads(case, (y,), (w,), i)


@pytest.mark.parametrize("case", _all("ssd"))
def test_ssd_scan(case):
    i = {k: _leaf(v) for k, v in case.ins.items()}
    o = case.opts
    Y, fin = orc.ssd_scan(i["X"], i["dt"], i["A"], i["B"], i["C"], o["chunk_size"], D=i.get("D"), z=i.get("z"),
                          dt_bias=i.get("dt_bias"), dt_softplus=o["dt_softplus"], initial_states=i.get("initial_states"),
                          return_final_states=True)
    heads = o.get("heads")
    if heads is not None:  # mamba-ssm vector: only the listed heads are exact (see make_fixtures.py)
        _close(Y[:, :, heads], case.outs["y"][:, :, heads], **tol(case))
        _close(fin[:, heads], case.outs["final_states"][:, heads], **tol(case))
        return
    _close(Y, case.outs["y"], **tol(case))
    _close(fin, case.outs["final_states"], **tol(case))
    _check_grads(case, (Y, fin), (i["grad_out"].detach(), i["grad_final_states"].detach()), i)


@pytest.mark.parametrize("case", _all("ssdvarlen"))
def test_ssd_scan_packed_sequences(case):
    """mamba-ssm's ``combined_varlen`` vector: cu_seqlens without seq_idx, so y runs through the boundary and only the
    states are per sequence (``seq_reset=False``)."""
    i = {k: v for k, v in case.ins.items()}
    o = case.opts
    Y, states = orc.ssd_scan(i["X"], i["dt"], i["A"], i["B"], i["C"], o["chunk_size"], dt_softplus=o["dt_softplus"],
                             cu_seqlens=i["cu_seqlens"], seq_reset=o["seq_reset"], return_varlen_states=True)
    heads = o["heads"]
    _close(Y[:, :, heads], case.outs["y"][:, :, heads], **tol(case))
    _close(states[:, heads], case.outs["varlen_states"][:, heads], **tol(case))


def test_ssd_scan_packed_sequences_restart():
    """With ``seq_reset`` a packed call equals the separate calls, sequence by sequence; an empty sequence has a zero state."""
    gen = torch.Generator().manual_seed(5)
    nl, nh, npj, nn = 11, 2, 3, 4
    X, dt = torch.randn(1, nl, nh, npj, generator=gen), torch.rand(1, nl, nh, generator=gen) * 0.5
    A, Bm, Cm = -torch.rand(nh, generator=gen) - 0.1, torch.randn(1, nl, 1, nn, generator=gen), torch.randn(1, nl, 1, nn, generator=gen)
    cu = torch.tensor([0, 4, 4, 9, 11])
    Y, fin, states = orc.ssd_scan(X, dt, A, Bm, Cm, 4, cu_seqlens=cu, return_final_states=True, return_varlen_states=True)
    assert states.shape == (4, nh, npj, nn) and float(states[1].abs().max()) == 0.0
    for k, (a, b) in enumerate(((0, 4), (4, 4), (4, 9), (9, 11))):
        if b == a:
            continue
        y_k, s_k = orc.ssd_scan(X[:, a:b], dt[:, a:b], A, Bm[:, a:b], Cm[:, a:b], 4, return_final_states=True)
        _close(Y[:, a:b], y_k, rtol=1e-6, atol=1e-6)
        _close(states[k], s_k[0], rtol=1e-6, atol=1e-6)
    _close(fin[0], states[-1], rtol=0, atol=0)
    with pytest.raises(ValueError):
        orc.ssd_scan(X, dt, A, Bm, Cm, 4, cu_seqlens=torch.tensor([0, 5, 10]))
