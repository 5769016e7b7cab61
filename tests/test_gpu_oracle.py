"""GPU parity against the CPU oracle on seeded inputs larger than the fixtures, plus
size-independent properties at the benchmark's full sizes."""

from __future__ import annotations

import pytest
import torch

from oracle import ssm_oracle as orc
from tests.gpu_util import FP32_TOL, HALF_TOL, REDUCED, close, leaf

pytestmark = pytest.mark.gpu


def _rand(gen, *shape, dtype=torch.float32, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(dtype)


def _tol(dtype):
    return FP32_TOL if dtype == torch.float32 else HALF_TOL


def _grad_check(outs_g, outs_o, weights, leaves_g, leaves_o, tol, tag):
    tot_g = sum((o.float() * w.cuda()).sum() for o, w in zip(outs_g, weights))
    tot_o = sum((o.float() * w).sum() for o, w in zip(outs_o, weights))
    keys = [k for k, v in leaves_g.items() if v is not None and v.requires_grad]
    gg = torch.autograd.grad(tot_g, [leaves_g[k] for k in keys], allow_unused=True)
    go = torch.autograd.grad(tot_o, [leaves_o[k] for k in keys], allow_unused=True)
    for k, a, b in zip(keys, gg, go):
        assert a is not None, f"{tag}: no gradient for {k}"
        close(a, b, **tol, what=f"{tag} d{k}", reduced=k in REDUCED)


SCAN_CASES = [
    # B, D, L, N, groups (0: (D,N), -1: (B,D,N)), dtype
    (2, 40, 200, 16, 1, torch.float32),
    (1, 36, 257, 16, 2, torch.float32),   # ragged length, two groups, rows not a multiple of the CTA tile
    (2, 8, 96, 128, 1, torch.float32),    # Mamba-2 sized state
    (1, 6, 70, 256, 1, torch.float32),    # largest supported state
    (2, 64, 128, 16, 1, torch.bfloat16),
    (2, 32, 120, 16, 32, torch.float16),  # per-channel time-varying B/C (upstream Mamba1 module layout)
    (2, 12, 45, 5, 0, torch.float32),
    (3, 10, 33, 24, -1, torch.float32),
    (1, 5, 64, 48, 1, torch.float32),
]


@pytest.mark.parametrize("nb,nd,nl,nn,groups,dtype", SCAN_CASES)
def test_selective_scan_matches_oracle(nb, nd, nl, nn, groups, dtype):
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(nb * 1000 + nd * 10 + nl)
    u = _rand(gen, nb, nd, nl, dtype=dtype)
    delta = _rand(gen, nb, nd, nl, dtype=dtype, scale=0.5)
    A = -torch.exp(_rand(gen, nd, nn, scale=0.5))
    shp = (nd, nn) if groups == 0 else (nb, nd, nn) if groups == -1 else (nb, groups, nn, nl)
    Bm, Cm = _rand(gen, *shp, dtype=dtype), _rand(gen, *shp, dtype=dtype)
    D, z, bias = _rand(gen, nd, dtype=dtype), _rand(gen, nb, nd, nl, dtype=dtype), _rand(gen, nd, dtype=dtype, scale=0.5)
    ins = dict(u=u, delta=delta, A=A, B=Bm, C=Cm, D=D, z=z, dt_bias=bias)
    lo = {k: v.clone().requires_grad_(True) for k, v in ins.items()}
    lg = {k: leaf(v) for k, v in ins.items()}
    yo, so = orc.selective_scan(lo["u"], lo["delta"], lo["A"], lo["B"], lo["C"], D=lo["D"], z=lo["z"], dt_bias=lo["dt_bias"],
                                softplus=True, return_last_state=True)
    yg, sg = ops.selective_scan(lg["u"], lg["delta"], lg["A"], lg["B"], lg["C"], D=lg["D"], z=lg["z"], dt_bias=lg["dt_bias"],
                                softplus=True, return_last_state=True)
    tol = _tol(dtype)
    close(yg, yo, **tol, what="out")
    close(sg, so, **tol, what="last_state")
    wy = _rand(gen, *yo.shape).to(dtype).float()
    ws = _rand(gen, *so.shape).to(dtype).float()
    _grad_check((yg, sg), (yo, so), (wy, ws), lg, lo, tol, "scan")


def test_selective_scan_minimal_and_empty():
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(5)
    u, delta = _rand(gen, 2, 3, 17), _rand(gen, 2, 3, 17).abs() * 0.3
    A, Bm, Cm = -torch.rand(3, 4, generator=gen), _rand(gen, 3, 4), _rand(gen, 3, 4)
    y = ops.selective_scan(u.cuda(), delta.cuda(), A.cuda(), Bm.cuda(), Cm.cuda())
    close(y, orc.selective_scan(u, delta, A, Bm, Cm), **FP32_TOL, what="minimal")
    y0, s0 = ops.selective_scan(u[:, :, :0].cuda(), delta[:, :, :0].cuda(), A.cuda(), Bm.cuda(), Cm.cuda(), return_last_state=True)
    assert y0.shape == (2, 3, 0) and float(s0.abs().max()) == 0.0
    with pytest.raises(ValueError):
        ops.selective_scan(u.cuda(), delta[:, :2].cuda(), A.cuda(), Bm.cuda(), Cm.cuda())
    with pytest.raises(ValueError):
        ops.selective_scan(u.cuda(), delta.cuda(), A.cuda(), Bm[:2].cuda(), Cm.cuda())


def test_selective_scan_initial_state_chains_at_full_size():
    """Splitting the sequence and passing the first half's final state as the second half's
    initial state reproduces the one-shot result (config: batch 8, D 1536, L 4096, N 16, bf16)."""
    from ssm_b200 import ops

    torch.manual_seed(0)
    nb, nd, nl, nn = 8, 1536, 4096, 16
    dev = "cuda"
    u = torch.randn(nb, nd, nl, device=dev, dtype=torch.bfloat16)
    delta = torch.randn(nb, nd, nl, device=dev, dtype=torch.bfloat16)
    A = -torch.exp(torch.randn(nd, nn, device=dev) * 0.5)
    Bm = torch.randn(nb, 1, nn, nl, device=dev, dtype=torch.bfloat16)
    Cm = torch.randn(nb, 1, nn, nl, device=dev, dtype=torch.bfloat16)
    D, z, bias = torch.randn(nd, device=dev), torch.randn(nb, nd, nl, device=dev, dtype=torch.bfloat16), torch.randn(nd, device=dev) - 2
    kw = dict(softplus=True, return_last_state=True, keep_state_fp32=True)
    y, s = ops.selective_scan(u, delta, A, Bm, Cm, D=D, z=z, dt_bias=bias, **kw)
    h = nl // 2
    y1, s1 = ops.selective_scan(u[..., :h], delta[..., :h], A, Bm[..., :h], Cm[..., :h], D=D, z=z[..., :h], dt_bias=bias, **kw)
    y2, s2 = ops.selective_scan(u[..., h:], delta[..., h:], A, Bm[..., h:], Cm[..., h:], D=D, z=z[..., h:], dt_bias=bias,
                                initial_state=s1, **kw)
    assert torch.equal(y[..., :h], y1)
    close(y2, y[..., h:], **HALF_TOL, what="second half")
    close(s2, s, **FP32_TOL, what="final state")
    # one batch row, a slice of channels, against the CPU oracle
    sl = slice(700, 716)
    yo, so = orc.selective_scan(u[0:1, sl, :512].cpu(), delta[0:1, sl, :512].cpu(), A[sl].cpu(), Bm[0:1, :, :, :512].cpu(),
                                Cm[0:1, :, :, :512].cpu(), D=D[sl].cpu(), z=z[0:1, sl, :512].cpu(), dt_bias=bias[sl].cpu(),
                                softplus=True, return_last_state=True)
    close(y[0:1, sl, :512], yo, **HALF_TOL, what="oracle slice")


STEP_CASES = [
    (4, 24, 16, 1, torch.float32), (3, 10, 5, 0, torch.float32), (2, 12, 128, 2, torch.float32),
    (8, 64, 16, 1, torch.bfloat16), (2, 6, 40, -1, torch.float16),
]


@pytest.mark.parametrize("nb,nd,nn,groups,dtype", STEP_CASES)
def test_state_step_matches_oracle(nb, nd, nn, groups, dtype):
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(nb * 100 + nd)
    state = _rand(gen, nb, nd, nn, scale=0.3)
    x, dt = _rand(gen, nb, nd, dtype=dtype), _rand(gen, nb, nd, dtype=dtype, scale=0.5)
    A = -torch.exp(_rand(gen, nd, nn, scale=0.5))
    shp = (nd, nn) if groups == 0 else (nb, nd, nn) if groups == -1 else (nb, groups, nn)
    Bm, Cm = _rand(gen, *shp, dtype=dtype), _rand(gen, *shp, dtype=dtype)
    D, z, bias = _rand(gen, nd, dtype=dtype), _rand(gen, nb, nd, dtype=dtype), _rand(gen, nd, dtype=dtype, scale=0.5)
    ins = dict(state=state, x=x, dt=dt, A=A, B=Bm, C=Cm, D=D, z=z, dt_bias=bias)
    tol = _tol(dtype)
    # three in-place steps, no gradients
    so, sg = state.clone(), state.clone().cuda()
    for _ in range(3):
        yo = orc.selective_state_step(so, x, dt, A, Bm, Cm, D=D, z=z, dt_bias=bias, softplus=True)
        yg = ops.selective_state_step(sg, x.cuda(), dt.cuda(), A.cuda(), Bm.cuda(), Cm.cuda(), D=D.cuda(), z=z.cuda(),
                                      dt_bias=bias.cuda(), softplus=True)
    close(yg, yo, **tol, what="y after 3 steps")
    close(sg, so, **tol, what="state after 3 steps")
    # gradients of one step, including through the new state
    lo = {k: v.clone().requires_grad_(True) for k, v in ins.items()}
    lg = {k: leaf(v) for k, v in ins.items()}
    yo, no = orc.selective_state_step(lo["state"], lo["x"], lo["dt"], lo["A"], lo["B"], lo["C"], D=lo["D"], z=lo["z"],
                                      dt_bias=lo["dt_bias"], softplus=True, inplace=False)
    from ssm_b200.ops import _StateStepFn

    yg, ng = _StateStepFn.apply(lg["state"], lg["x"], lg["dt"], lg["A"], lg["B"], lg["C"], lg["D"], lg["z"], lg["dt_bias"], True)
    wy, wn = _rand(gen, nb, nd).to(dtype).float(), _rand(gen, nb, nd, nn)
    _grad_check((yg, ng), (yo, no), (wy, wn), lg, lo, tol, "step")


def test_state_step_heads_matches_flattened_oracle():
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(7)
    nb, nh, npj, nn, g = 3, 4, 8, 128, 2
    state = _rand(gen, nb, nh, npj, nn, scale=0.3)
    x, z = _rand(gen, nb, nh, npj, dtype=torch.bfloat16), _rand(gen, nb, nh, npj, dtype=torch.bfloat16)
    dt = _rand(gen, nb, nh, dtype=torch.bfloat16, scale=0.5)
    A, D, bias = -torch.exp(_rand(gen, nh, scale=0.5)), _rand(gen, nh), _rand(gen, nh, scale=0.5)
    Bm, Cm = _rand(gen, nb, g, nn, dtype=torch.bfloat16), _rand(gen, nb, g, nn, dtype=torch.bfloat16)
    so = state.reshape(nb, nh * npj, nn).clone()
    rep = lambda v: v[:, None].expand(nh, npj).reshape(-1)  # noqa: E731
    yo = orc.selective_state_step(so, x.reshape(nb, -1), dt.float().repeat_interleave(npj, dim=1).to(torch.bfloat16),
                                  A[:, None, None].expand(nh, npj, nn).reshape(nh * npj, nn), Bm, Cm, D=rep(D),
                                  z=z.reshape(nb, -1), dt_bias=rep(bias), softplus=True)
    sg = state.clone().cuda()
    yg = ops.selective_state_step_heads(sg, x.cuda(), dt.cuda(), A.cuda(), Bm.cuda(), Cm.cuda(), D=D.cuda(), z=z.cuda(),
                                        dt_bias=bias.cuda(), softplus=True)
    close(yg.reshape(nb, -1), yo, **HALF_TOL, what="y")
    close(sg.reshape(nb, nh * npj, nn), so, **FP32_TOL, what="state")


def test_conv_update_matches_full_conv():
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(11)
    nb, nc, k, nl = 3, 20, 4, 9
    x = _rand(gen, nb, nc, nl)
    w, b = torch.rand(nc, k, generator=gen) - 0.5, _rand(gen, nc, scale=0.2)
    full = orc.dw_causal_conv(x, w, b, "silu")
    cs = torch.zeros(nb, nc, k).cuda()
    for t in range(nl):
        y = ops.dw_causal_conv_update(cs, x[:, :, t].contiguous().cuda(), w.cuda(), b.cuda(), "silu")
        close(y, full[:, :, t], **FP32_TOL, what=f"t={t}")


CHUNK_CASES = [
    (2, 100, 3, 16, 32, "blhp", torch.float32, None), (2, 64, 2, 8, 16, "hp", torch.float32, [64, 20]),
    (1, 130, 4, 32, 64, "bhp", torch.float32, None), (2, 96, 2, 64, 32, "blhp", torch.bfloat16, [50, 96]),
    # 16-bit per-token B / C / z: the 16-byte-lane kernels.  Three threads per head (no shuffle reduction) and ragged lengths;
    # one piece in the backward but several in the forward; sixteen threads per head and a chunk that ends inside a load batch
    (2, 150, 5, 24, 48, "blhp", torch.float16, [150, 7]), (1, 77, 3, 8, 200, "blhp", torch.bfloat16, None),
    (2, 131, 2, 128, 33, "blhp", torch.bfloat16, [131, 65]),
    # more than 64 pieces: the carry over the pieces runs several passes of its four groups
    (1, 1100, 2, 8, 7, "hp", torch.float32, None),
]


@pytest.mark.parametrize("nb,nl,nh,npj,chunk,layout,dtype,lens", CHUNK_CASES)
def test_chunk_scan_matches_oracle(nb, nl, nh, npj, chunk, layout, dtype, lens):
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(nl * 7 + npj)
    X = _rand(gen, nb, nl, nh, npj, dtype=dtype)
    dt = (torch.rand(nb, nl, nh, generator=gen) * 0.5 + 0.01).to(dtype)
    A = -torch.exp(_rand(gen, nh, npj, scale=0.5))
    shp = {"hp": (nh, npj), "bhp": (nb, nh, npj), "blhp": (nb, nl, nh, npj)}[layout]
    Bm, Cm = _rand(gen, *shp, dtype=dtype), _rand(gen, *shp, dtype=dtype)
    D, z, init = _rand(gen, nh, dtype=dtype), _rand(gen, nb, nl, nh, npj, dtype=dtype), _rand(gen, nb, nh, npj, dtype=dtype, scale=0.5)
    meta = None if lens is None else {"seq_lens": lens}
    ins = dict(X=X, dt=dt, A=A, B=Bm, C=Cm, D=D, z=z, initial_states=init)
    lo = {k: v.clone().requires_grad_(True) for k, v in ins.items()}
    lg = {k: leaf(v) for k, v in ins.items()}
    Yo = orc.ssd_chunk_scan(lo["X"], lo["dt"], lo["A"], lo["B"], lo["C"], chunk, D=lo["D"], z=lo["z"], seq_meta=meta,
                            initial_states=lo["initial_states"])
    Yg = ops.ssd_chunk_scan(lg["X"], lg["dt"], lg["A"], lg["B"], lg["C"], chunk, D=lg["D"], z=lg["z"], seq_meta=meta,
                            initial_states=lg["initial_states"])
    tol = _tol(dtype)
    close(Yg, Yo, **tol, what="Y")
    # the chunk size is not allowed to matter
    Y1 = ops.ssd_chunk_scan(lg["X"], lg["dt"], lg["A"], lg["B"], lg["C"], nl + 5, D=lg["D"], z=lg["z"], seq_meta=meta,
                            initial_states=lg["initial_states"])
    close(Y1, Yg, **tol, what="chunk-size invariance")
    w = _rand(gen, *Yo.shape).to(dtype).float()
    _grad_check((Yg,), (Yo,), (w,), lg, lo, tol, "chunk")


CONV_CASES = [
    (2, 24, 200, 4, True, "silu", torch.float32), (2, 24, 200, 4, False, "silu", torch.float32),
    (1, 7, 131, 3, True, "identity", torch.float32), (2, 10, 77, 7, False, "silu", torch.float32),
    (2, 64, 256, 4, True, "silu", torch.bfloat16), (2, 64, 256, 4, False, "silu", torch.bfloat16),
    (1, 16, 40, 8, True, "swish", torch.float16), (3, 9, 5, 2, False, "none", torch.float32),
    (2, 12, 64, 7, True, "silu", torch.float32),   # channels-first, 16-byte accesses, taps reaching two vectors back
    (2, 12, 72, 8, True, "silu", torch.bfloat16),  # widest kernel, length a multiple of the vector but not of the block
]


@pytest.mark.parametrize("nb,nc,nl,k,first,act,dtype", CONV_CASES)
def test_conv_matches_oracle(nb, nc, nl, k, first, act, dtype):
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(nc * 31 + nl + k)
    x = _rand(gen, *((nb, nc, nl) if first else (nb, nl, nc)), dtype=dtype)
    w = (torch.rand(nc, k, generator=gen) - 0.5).to(dtype)
    b = _rand(gen, nc, dtype=dtype, scale=0.3)
    ins = dict(x=x, weight=w, bias=b)
    lo = {k_: v.clone().requires_grad_(True) for k_, v in ins.items()}
    lg = {k_: leaf(v) for k_, v in ins.items()}
    yo = orc.dw_causal_conv(lo["x"], lo["weight"], lo["bias"], act)
    yg = ops.dw_causal_conv(lg["x"], lg["weight"], lg["bias"], act)
    tol = _tol(dtype)
    close(yg, yo, **tol, what="y")
    wy = _rand(gen, *yo.shape).to(dtype).float()
    _grad_check((yg,), (yo,), (wy,), lg, lo, tol, "conv")


def test_conv_halo_splits_a_sequence():
    from ssm_b200 import ops

    torch.manual_seed(3)
    nb, nc, nl, k = 2, 48, 512, 4
    x = torch.randn(nb, nc, nl, device="cuda", dtype=torch.bfloat16)
    w, b = torch.rand(nc, k, device="cuda") - 0.5, torch.randn(nc, device="cuda") * 0.1
    y = ops.dw_causal_conv(x, w, b, "silu")
    h = 256
    y1 = ops.dw_causal_conv(x[..., :h].contiguous(), w, b, "silu")
    y2 = ops.dw_causal_conv(x[..., h:].contiguous(), w, b, "silu", halo=x[..., h - (k - 1):h].float().contiguous())
    assert torch.equal(torch.cat([y1, y2], dim=-1), y)


def test_conv_halo_backward_matches_the_unsplit_sequence():
    from ssm_b200 import ops

    torch.manual_seed(5)
    nb, nc, nl, k, h = 2, 24, 384, 4, 128
    x = torch.randn(nb, nc, nl, device="cuda")
    w, b = (torch.rand(nc, k, device="cuda") - 0.5), torch.randn(nc, device="cuda") * 0.1
    gy = torch.randn(nb, nc, nl, device="cuda")
    xf, wf, bf = (t.clone().requires_grad_(True) for t in (x, w, b))
    ops.dw_causal_conv(xf, wf, bf, "silu").backward(gy)
    x1, x2 = x[..., :h].contiguous().requires_grad_(True), x[..., h:].contiguous().requires_grad_(True)
    w2, b2 = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    y1 = ops.dw_causal_conv(x1, w2, b2, "silu")
    y2 = ops.dw_causal_conv(x2, w2, b2, "silu", halo=x[..., h - (k - 1):h].contiguous())
    (y1 * gy[..., :h]).sum().add((y2 * gy[..., h:]).sum()).backward()
    close(x2.grad, xf.grad[..., h:], **FP32_TOL, what="dx of the second shard")
    # the first shard's last K-1 inputs also feed the second shard's outputs; that part flows through the halo
    close(x1.grad[..., : h - (k - 1)], xf.grad[..., : h - (k - 1)], **FP32_TOL, what="dx of the first shard")
    close(w2.grad, wf.grad, **FP32_TOL, what="dweight")
    close(b2.grad, bf.grad, **FP32_TOL, what="dbias")


NORM_CASES = [
    (3, 50, 768, torch.float32, torch.float32), (2, 33, 768, torch.bfloat16, torch.float32),
    (2, 20, 2560, torch.bfloat16, torch.bfloat16), (2, 9, 5120, torch.float16, torch.float32),
    (2, 7, 100, torch.float32, None), (1, 5, 33, torch.float32, torch.float32), (1, 4, 16384, torch.bfloat16, torch.float32),
]


@pytest.mark.parametrize("is_rms", [False, True])
@pytest.mark.parametrize("prenorm", [True, False])
@pytest.mark.parametrize("nb,nl,nd,dtype,rdtype", NORM_CASES)
def test_norm_matches_oracle(nb, nl, nd, dtype, rdtype, prenorm, is_rms):
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(nd + nl)
    x, w, b = _rand(gen, nb, nl, nd, dtype=dtype), _rand(gen, nd, dtype=dtype), _rand(gen, nd, dtype=dtype)
    res = None if rdtype is None else _rand(gen, nb, nl, nd, dtype=rdtype)
    ins = dict(x=x, weight=w, bias=b, residual=res)
    lo = {k: (None if v is None else v.clone().requires_grad_(True)) for k, v in ins.items()}
    lg = {k: leaf(v) for k, v in ins.items()}
    yo, ro = orc.fused_layer_norm(lo["x"], lo["weight"], lo["bias"], residual=lo["residual"], is_rms=is_rms, prenorm=prenorm,
                                  return_residual=True)
    yg, rg = ops.fused_layer_norm(lg["x"], lg["weight"], lg["bias"], residual=lg["residual"], is_rms=is_rms, prenorm=prenorm,
                                  return_residual=True)
    tol = _tol(dtype)
    close(yg, yo, **tol, what="y")
    close(rg, ro, **FP32_TOL, what="residual_out")
    wy = _rand(gen, *yo.shape).to(dtype).float()
    _grad_check((yg,), (yo,), (wy,), lg, lo, tol, "norm")


def test_channel_major_row_layout_matches_dense():
    """(D, B, L) buffers viewed as (B, D, L) are addressed in place by the scan and the conv (forward
    and backward) and give the dense-layout results."""
    from ssm_b200 import ops

    torch.manual_seed(5)
    nb, nd, nl, nn = 3, 40, 200, 16
    dev = "cuda"

    def cm(*shape, dtype=torch.bfloat16):  # channel-major buffer, (B, D, L) view
        return torch.randn(shape[1], shape[0], shape[2], device=dev, dtype=dtype).permute(1, 0, 2)

    u, delta, z, go = cm(nb, nd, nl), cm(nb, nd, nl), cm(nb, nd, nl), cm(nb, nd, nl)
    assert not u.is_contiguous()
    A = -torch.exp(torch.randn(nd, nn, device=dev) * 0.5)
    Bm, Cm = torch.randn(nb, 1, nn, nl, device=dev, dtype=torch.bfloat16), torch.randn(nb, 1, nn, nl, device=dev, dtype=torch.bfloat16)
    D, bias = torch.randn(nd, device=dev), torch.randn(nd, device=dev) * 0.5
    w = torch.rand(nd, 4, device=dev) - 0.5

    def run(tensors):
        uu, dd, zz, gg = (t.clone().requires_grad_(True) if i < 3 else t for i, t in enumerate(tensors))
        x = ops.dw_causal_conv(uu, w, None, "silu")
        y, s = ops.selective_scan(x, dd, A, Bm, Cm, D=D, z=zz, dt_bias=bias, softplus=True, return_last_state=True)
        y.backward(gg)
        return y, s, uu.grad, dd.grad, zz.grad

    got = run((u, delta, z, go))
    want = run(tuple(t.contiguous() for t in (u, delta, z, go)))
    assert got[0].stride() == u.stride()  # the output keeps the layout of its input
    for g_, w_, name in zip(got, want, ("y", "state", "du", "ddelta", "dz")):
        assert torch.equal(g_.contiguous(), w_.contiguous()), name
