"""GPU parity against the golden fixtures (upstream's own vectors and recorded runs of
upstream's Python operators): outputs, final states and gradients, through the C ABI.

Vectors that carry their own bar (``rtol`` in the case options: upstream's stored known-answer files, whose bars are
tighter than the fp32 bar used elsewhere) are judged with the absolute term scaled by the tensor's magnitude."""

from __future__ import annotations

import pytest
import torch

from tests.fixtures import cases, tol
from tests.gpu_util import REDUCED, close, dev, leaf

pytestmark = pytest.mark.gpu

PACKS = ("upstream_kats", "reference_runs")


def _all(family):
    return [pytest.param(c, id=f"{p}:{c.name}") for p in PACKS for c in cases(p, family)]


def _grads(case, outs, weights, leaves):
    if not case.grads:
        return
    live = {k: v for k, v in leaves.items() if v is not None and k in case.grads and v.requires_grad}
    total = sum((o.float() * w.float().cuda()).sum() for o, w in zip(outs, weights))
    got = torch.autograd.grad(total, list(live.values()), allow_unused=True)
    for (k, _), g in zip(live.items(), got):
        assert g is not None, f"no gradient for {k}"
        close(g, case.grads[k], **tol(case, grad=True), what=f"{case.name} d{k}", reduced=k in REDUCED or "rtol" in case.opts)


@pytest.mark.parametrize("case", _all("scan"))
def test_selective_scan(case):
    from ssm_b200 import ops

    i = {k: leaf(v) for k, v in case.ins.items()}
    y, last = ops.selective_scan(i["u"], i["delta"], i["A"], i["B"], i["C"], D=i.get("D"), z=i.get("z"),
                                 dt_bias=i.get("dt_bias"), softplus=case.opts["softplus"], return_last_state=True)
    assert y.dtype == i["u"].dtype and last.dtype == i["u"].dtype
    close(y, case.outs["out"], **tol(case), what=f"{case.name} out", reduced="rtol" in case.opts)
    if "last_state" in case.outs:
        close(last, case.outs["last_state"], **tol(case), what=f"{case.name} last_state", reduced="rtol" in case.opts)
    if "grad_out" in case.ins:
        _grads(case, (y, last), (case.ins["grad_out"], case.ins["grad_last_state"]), i)
    else:
        _grads(case, (y,), (torch.ones_like(y),), i)


@pytest.mark.parametrize("case", _all("step"))
def test_selective_state_step(case):
    from ssm_b200 import ops

    i = {k: leaf(v, grad=False) for k, v in case.ins.items()}
    y = ops.selective_state_step(i["state"], i["x"], i["dt"], i["A"], i["B"], i["C"], D=i.get("D"), z=i.get("z"),
                                 dt_bias=i.get("dt_bias"), softplus=case.opts["softplus"])
    close(y, case.outs["y"], **tol(case), what=f"{case.name} y", reduced="rtol" in case.opts)
    close(i["state"], case.outs["state"], **tol(case), what=f"{case.name} state", reduced="rtol" in case.opts)


@pytest.mark.parametrize("case", _all("chunk"))
def test_ssd_chunk_scan(case):
    from ssm_b200 import ops

    i = {k: leaf(v) for k, v in case.ins.items()}
    meta = None
    if "cu_seqlens" in i:
        meta = {"cu_seqlens": i["cu_seqlens"]}
    elif "seq_lens" in i:
        meta = {"seq_lens": i["seq_lens"]}
    Y = ops.ssd_chunk_scan(i["X"], i["dt"], i["A"], i["B"], i["C"], case.opts["chunk_size"], D=i.get("D"), z=i.get("z"),
                           seq_meta=meta, initial_states=i.get("initial_states"))
    close(Y, case.outs["Y"], **tol(case), what=f"{case.name} Y", reduced="rtol" in case.opts)
    if "grad_out" in case.ins:
        _grads(case, (Y,), (case.ins["grad_out"],), i)


@pytest.mark.parametrize("case", _all("conv"))
def test_dw_causal_conv(case):
    from ssm_b200 import ops

    i = {k: leaf(v) for k, v in case.ins.items()}
    y = ops.dw_causal_conv(i["x"], i["weight"], bias=i.get("bias"), activation=case.opts["activation"])
    assert y.shape == i["x"].shape and y.dtype == i["x"].dtype
    close(y, case.outs["y"], **tol(case), what=f"{case.name} y", reduced="rtol" in case.opts)
    w = case.ins["grad_out"] if "grad_out" in case.ins else torch.ones_like(y)
    _grads(case, (y,), (w,), i)


@pytest.mark.parametrize("case", _all("norm"))
def test_fused_layer_norm(case):
    from ssm_b200 import ops

    i = {k: leaf(v) for k, v in case.ins.items()}
    o = case.opts
    y, res = ops.fused_layer_norm(i["x"], i["weight"], i.get("bias"), residual=i.get("residual"), is_rms=o["is_rms"],
                                  eps=o["eps"], prenorm=o["prenorm"], residual_in_fp32=o.get("residual_in_fp32", True),
                                  return_residual=True)
    close(y, case.outs["y"], **tol(case), what=f"{case.name} y", reduced="rtol" in case.opts)
    if "residual_out" in case.outs:
        close(res, case.outs["residual_out"], **tol(case), what=f"{case.name} residual_out", reduced="rtol" in case.opts)
    w = case.ins["grad_out"] if "grad_out" in case.ins else torch.ones_like(y)
    _grads(case, (y,), (w,), i)


@pytest.mark.parametrize("case", _all("ssd"))
def test_ssd_scan(case):
    from ssm_b200 import ops

    i = {k: leaf(v) for k, v in case.ins.items()}
    o = case.opts
    Y, fin = ops.ssd_scan(i["X"], i["dt"], i["A"], i["B"], i["C"], o["chunk_size"], D=i.get("D"), z=i.get("z"),
                          dt_bias=i.get("dt_bias"), dt_softplus=o["dt_softplus"], initial_states=i.get("initial_states"),
                          return_final_states=True)
    heads = o.get("heads")
    if heads is not None:  # mamba-ssm vector: only the listed heads follow the exact recurrence
        close(Y[:, :, heads], case.outs["y"][:, :, heads], **tol(case), what=f"{case.name} y", reduced="rtol" in case.opts)
        close(fin[:, heads], case.outs["final_states"][:, heads], **tol(case), what=f"{case.name} final", reduced="rtol" in case.opts)
        return
    close(Y, case.outs["y"], **tol(case), what=f"{case.name} y", reduced="rtol" in case.opts)
    close(fin, case.outs["final_states"], **tol(case), what=f"{case.name} final", reduced="rtol" in case.opts)
    _grads(case, (Y, fin), (case.ins["grad_out"], case.ins["grad_final_states"]), i)


@pytest.mark.parametrize("case", _all("ssdvarlen"))
def test_ssd_scan_packed_sequences(case):
    """mamba-ssm's ``combined_varlen`` vector (cu_seqlens without seq_idx: y runs through the boundary, states per sequence)."""
    from ssm_b200 import ops

    i = {k: dev(v) for k, v in case.ins.items()}
    o = case.opts
    Y, states = ops.ssd_scan(i["X"], i["dt"], i["A"], i["B"], i["C"], o["chunk_size"], dt_softplus=o["dt_softplus"],
                             cu_seqlens=i["cu_seqlens"], seq_reset=o["seq_reset"], return_varlen_states=True)
    heads = o["heads"]
    close(Y[:, :, heads], case.outs["y"][:, :, heads], **tol(case), what=f"{case.name} y", reduced=True)
    close(states[:, heads], case.outs["varlen_states"][:, heads], **tol(case), what=f"{case.name} varlen states", reduced=True)
