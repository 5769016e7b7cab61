"""CUDA path against the CPU oracle at the sizes the benchmark configurations state.

Where the oracle can run the whole configuration (the fp32 prefill scan, the decode step) it
does; for the long state-space-dual scans the operator runs at the full size -- so the grids
and heads-per-CTA splits are the ones the benchmark launches -- and one batch row x two heads
x every time step is compared with the stepping oracle on exactly those slices.
"""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from oracle import ssm_oracle as orc
from tests.gpu_util import FP32_TOL, HALF_TOL, REDUCED, close, close_sum

pytestmark = pytest.mark.gpu

SSD_TOL = dict(rtol=2e-2, atol=2e-2)  # 256-term bf16 product sums: absolute term scaled by the tensor's magnitude


def test_prefill_scan_fp32_whole_configuration():
    """selective_scan forward: batch 1, d_inner 512, seqlen 2048, d_state 16, fp32, B / C shared by all channels,
    D skip, SiLU(z) gate, softplus inside the operator; output and final state (seed 0)."""
    from ssm_b200 import ops

    torch.manual_seed(0)
    nb, nd, nl, nn = 1, 512, 2048, 16
    u = torch.randn(nb, nd, nl)
    delta = F.softplus(torch.randn(nb, nd, nl) - 2)
    A = -torch.exp(torch.randn(nd, nn) * 0.5)
    Bm, Cm = torch.randn(nb, 1, nn, nl), torch.randn(nb, 1, nn, nl)
    D, z = torch.randn(nd), torch.randn(nb, nd, nl)
    yo, so = orc.selective_scan(u, delta, A, Bm, Cm, D=D, z=z, softplus=True, return_last_state=True)
    yg, sg = ops.selective_scan(u.cuda(), delta.cuda(), A.cuda(), Bm.cuda(), Cm.cuda(), D=D.cuda(), z=z.cuda(), softplus=True,
                                return_last_state=True)
    close(yg, yo, **FP32_TOL, what="y")
    close(sg, so, **FP32_TOL, what="final state")


def test_prefill_scan_fp32_gradients_whole_configuration():
    """The same configuration backward: all eight gradients, with a final-state term in the loss."""
    from ssm_b200 import ops

    torch.manual_seed(0)
    nb, nd, nl, nn = 1, 512, 2048, 16
    ins = dict(u=torch.randn(nb, nd, nl), delta=torch.randn(nb, nd, nl) - 2, A=-torch.exp(torch.randn(nd, nn) * 0.5),
               B=torch.randn(nb, 1, nn, nl), C=torch.randn(nb, 1, nn, nl), D=torch.randn(nd), z=torch.randn(nb, nd, nl),
               dt_bias=torch.randn(nd) * 0.3)
    wy, ws = torch.randn(nb, nd, nl), torch.randn(nb, nd, nn)
    lo = {k: v.clone().requires_grad_(True) for k, v in ins.items()}
    lg = {k: v.clone().cuda().requires_grad_(True) for k, v in ins.items()}

    def run(ops_, t, dev):
        y, s = ops_.selective_scan(t["u"], t["delta"], t["A"], t["B"], t["C"], D=t["D"], z=t["z"], dt_bias=t["dt_bias"], softplus=True,
                                   return_last_state=True)
        return torch.autograd.grad((y * wy.to(dev)).sum() + (s * ws.to(dev)).sum(), list(t.values()))

    for k, a, b in zip(ins, run(ops, lg, "cuda"), run(orc, lo, "cpu")):
        close(a, b, **FP32_TOL, what=f"d{k}", reduced=k in REDUCED)


def _ssd_inputs(nb, nl, nh, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    bf = torch.bfloat16
    kw = dict(generator=g, device="cuda")
    t = dict(
        X=torch.randn(nb, nl, nh, 64, **kw).to(bf), dt=(torch.randn(nb, nl, nh, **kw) - 3).to(bf),
        B=(torch.randn(nb, nl, 1, 128, **kw) / 128 ** 0.5).to(bf), C=(torch.randn(nb, nl, 1, 128, **kw) / 128 ** 0.5).to(bf),
        z=torch.randn(nb, nl, nh, 64, **kw).to(bf), A=-torch.exp(torch.rand(nh, **kw) * 2.7726), D=torch.randn(nh, **kw))
    return t


def _ssd_slice_oracle(t, b, heads, init=None, bias=None):
    hs = torch.tensor(heads)
    c = lambda v: v.cpu()  # noqa: E731
    return orc.ssd_scan(c(t["X"][b:b + 1][:, :, heads]), c(t["dt"][b:b + 1][:, :, heads]), c(t["A"])[hs], c(t["B"][b:b + 1]), c(t["C"][b:b + 1]), 256,
                        D=c(t["D"])[hs], z=c(t["z"][b:b + 1][:, :, heads]), dt_bias=None if bias is None else c(bias)[hs], dt_softplus=True,
                        initial_states=None if init is None else c(init[b:b + 1][:, heads]), return_final_states=True)


def test_ssd_chunk_scan_configuration_on_head_slices():
    """Batch 8, seqlen 8192, 48 heads x 64, d_state 128, one group, chunk 256, bf16: the operator at full size
    (twelve heads per scan CTA), one batch row x two heads x all 8192 steps against the stepping oracle."""
    from ssm_b200 import ops

    t = _ssd_inputs(8, 8192, 48, seed=0)
    assert ops.ssd_tensor_core_supported(t["X"], t["B"], 256)
    Y, S = ops.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 256, D=t["D"], z=t["z"], dt_softplus=True, return_final_states=True,
                        check_status=True)
    assert S.shape == (8, 48, 64, 128) and S.dtype == torch.float32
    for b, heads in ((3, [5, 40]), (7, [47, 0])):
        Yo, So = _ssd_slice_oracle(t, b, heads)
        close(Y[b:b + 1][:, :, heads], Yo, **SSD_TOL, what=f"Y row {b} heads {heads}", reduced=True)
        close(S[b:b + 1][:, heads], So, **SSD_TOL, what=f"final state row {b} heads {heads}", reduced=True)


def test_ssd_long_shard_shape_direct_and_two_phase():
    """Batch 2, 80 heads x 64, d_state 128, a 16384-token shard (what one of eight ranks holds of a 131072-token
    sequence; two heads per state CTA): direct call and the state-phase / finish-phase split with an incoming state."""
    from ssm_b200 import ops

    nb, nl, nh = 2, 16384, 80
    t = _ssd_inputs(nb, nl, nh, seed=1)
    g = torch.Generator(device="cuda").manual_seed(2)
    init = torch.randn(nb, nh, 64, 128, generator=g, device="cuda") * 0.5
    bias = torch.randn(nh, generator=g, device="cuda") * 0.3
    Y, S = ops.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 256, D=t["D"], z=t["z"], dt_bias=bias, dt_softplus=True,
                        initial_states=init, return_final_states=True, check_status=True)
    heads = [0, 79]
    Yo, So = _ssd_slice_oracle(t, 1, heads, init=init, bias=bias)
    close(Y[1:2][:, :, heads], Yo, **SSD_TOL, what="Y", reduced=True)
    close(S[1:2][:, heads], So, **SSD_TOL, what="final state", reduced=True)
    w = ops._SsdWorkspace(t["X"], t["dt"], t["A"], t["B"], t["C"], t["D"], t["z"], bias, True, 256)
    w.run(1, None, False)
    Y2, S2 = w.run(2, init, True)
    ops.ssd_check_status()
    close(Y2, Y, **SSD_TOL, what="two-phase Y", reduced=True)
    close(S2, S, **SSD_TOL, what="two-phase final state", reduced=True)


SSD_GRAD_CASES = [
    # batch, len, heads, groups, dtype, gate, initial state, D per (head, p)
    pytest.param(1, 384, 2, 1, torch.bfloat16, True, True, False, id="L384-pad-z-init"),
    pytest.param(2, 1024, 4, 2, torch.bfloat16, True, True, False, id="L1024-groups-z-init"),
    pytest.param(1, 512, 2, 2, torch.bfloat16, False, False, False, id="L512-plain"),
    pytest.param(1, 700, 4, 1, torch.float16, True, True, True, id="L700-fp16-Dhp"),
]


@pytest.mark.parametrize("backward", ["dual", "scan"])
@pytest.mark.parametrize("nb,nl,nh,ng,dtype,use_z,use_init,d_hp", SSD_GRAD_CASES)
def test_ssd_gradients_at_the_tensor_core_shape(nb, nl, nh, ng, dtype, use_z, use_init, d_hp, backward):
    """headdim 64 / d_state 128, 16-bit operands: every gradient of ssd_scan (dX, ddt, dA, dB, dC, dD, dz, ddt_bias, dinitial)
    against the oracle's autograd, with a final-state term in the loss.  ``scan`` = fp32 selective-scan kernels on the
    flattened channels (element-wise bars); ``dual`` = the chunked GEMM form on the tensor cores (every gradient is a
    16-bit-operand contraction: the tensor-core bar; the decay-path sums dA and ddt_bias against the sum of their terms'
    magnitudes, ddt with the absolute term at 5 % of its largest entry, since it holds |A| times the 0.3 % noise of
    <adjoint state, state>)."""
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(17 + nl)
    ins = dict(X=torch.randn(nb, nl, nh, 64, generator=gen).to(dtype), dt=(torch.randn(nb, nl, nh, generator=gen) - 3).to(dtype),
               A=-torch.exp(torch.rand(nh, generator=gen) * 2.77), B=(torch.randn(nb, nl, ng, 128, generator=gen) / 128 ** 0.5).to(dtype),
               C=(torch.randn(nb, nl, ng, 128, generator=gen) / 128 ** 0.5).to(dtype),
               D=torch.randn(nh, 64, generator=gen) if d_hp else torch.randn(nh, generator=gen),
               z=torch.randn(nb, nl, nh, 64, generator=gen).to(dtype) if use_z else None, dt_bias=torch.randn(nh, generator=gen) * 0.3,
               initial_states=torch.randn(nb, nh, 64, 128, generator=gen) * 0.5 if use_init else None)
    wy = torch.randn(nb, nl, nh, 64, generator=gen).to(dtype).float()
    wf = torch.randn(nb, nh, 64, 128, generator=gen)
    names = [k for k, v in ins.items() if v is not None]
    lo = {k: (None if v is None else v.clone().requires_grad_(True)) for k, v in ins.items()}
    lg = {k: (None if v is None else v.clone().cuda().requires_grad_(True)) for k, v in ins.items()}
    assert ops.ssd_tensor_core_supported(lg["X"], lg["B"], 256)

    def run(ops_, t, dev, **kw):
        Y, fin = ops_.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 256, D=t["D"], z=t["z"], dt_bias=t["dt_bias"], dt_softplus=True,
                               initial_states=t["initial_states"], return_final_states=True, **kw)
        return Y, fin, torch.autograd.grad((Y.float() * wy.to(dev)).sum() + (fin * wf.to(dev)).sum(), [t[k] for k in names])

    Yg, Sg, gg = run(ops, lg, "cuda", backward=backward)
    ops.ssd_check_status()
    Yo, So, go = run(orc, lo, "cpu")
    close(Yg, Yo, **SSD_TOL, what="Y", reduced=True)
    close(Sg, So, **SSD_TOL, what="final state", reduced=True)
    want = dict(zip(names, go))
    for k, a in zip(names, gg):
        b = want[k]
        if backward == "scan":
            # ddt sums 64 rounded per-channel terms per (token, head): a contraction like the parameter gradients
            close(a, b, **HALF_TOL, what=f"d{k}", reduced=k in REDUCED or k == "dt")
        elif k in ("A", "dt_bias"):
            pre = ins["dt"].float() + ins["dt_bias"]
            delta, sig = torch.nn.functional.softplus(pre), torch.sigmoid(pre)
            draw = want["dt"].float()
            terms = draw.abs().sum((0, 1)) if k == "dt_bias" else (delta * draw.abs() / sig).sum((0, 1)) / ins["A"].abs()
            close_sum(a, b, terms, 5e-2, what=f"d{k}")
        elif k == "dt":
            close(a, b, rtol=2e-2, atol=5e-2, what="ddt", reduced=True)
        else:
            close(a, b, **SSD_TOL, what=f"d{k}", reduced=True)


def test_ssd_packed_sequences_on_the_tensor_cores():
    """Three sequences (one of them empty) packed along L at headdim 64 / d_state 128: outputs, per-sequence states and
    the gradients of X, B, C and z against the oracle; every sequence runs as its own tensor-core scan."""
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(23)
    nl, nh = 900, 2
    bf = torch.bfloat16
    ins = dict(X=torch.randn(1, nl, nh, 64, generator=gen).to(bf), dt=(torch.randn(1, nl, nh, generator=gen) - 3).to(bf),
               A=-torch.exp(torch.rand(nh, generator=gen) * 2.77), B=(torch.randn(1, nl, 1, 128, generator=gen) / 128 ** 0.5).to(bf),
               C=(torch.randn(1, nl, 1, 128, generator=gen) / 128 ** 0.5).to(bf), D=torch.randn(nh, generator=gen),
               z=torch.randn(1, nl, nh, 64, generator=gen).to(bf))
    cu = torch.tensor([0, 300, 300, 812, 900])
    wy = torch.randn(1, nl, nh, 64, generator=gen).to(bf).float()
    ws = torch.randn(4, nh, 64, 128, generator=gen)
    names = ["X", "B", "C", "z"]

    def run(ops_, t, dev_):
        Y, st = ops_.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 256, D=t["D"], z=t["z"], dt_softplus=True,
                              cu_seqlens=cu.to(dev_), return_varlen_states=True)
        return Y, st, torch.autograd.grad((Y.float() * wy.to(dev_)).sum() + (st * ws.to(dev_)).sum(), [t[k] for k in names])

    lo = {k: v.clone().requires_grad_(k in names) for k, v in ins.items()}
    lg = {k: v.clone().cuda().requires_grad_(k in names) for k, v in ins.items()}
    Yg, Sg, gg = run(ops, lg, "cuda")
    ops.ssd_check_status()
    Yo, So, go = run(orc, lo, "cpu")
    close(Yg, Yo, **SSD_TOL, what="Y", reduced=True)
    close(Sg, So, **SSD_TOL, what="varlen states", reduced=True)
    assert float(Sg[1].detach().abs().max()) == 0.0
    for k, a, b in zip(names, gg, go):
        close(a, b, **SSD_TOL, what=f"d{k}", reduced=True)


def test_decode_step_configuration():
    """One Mamba-1 decode step at batch 256, d_inner 5120, d_state 16 (fp32 state, bf16 activations, B / C shared by the
    channels of a row) with the conv-window update in front of it, whole configuration against the oracle."""
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(4)
    nb, nd, nn, k = 256, 5120, 16, 4
    bf = torch.bfloat16
    state = torch.randn(nb, nd, nn, generator=gen) * 0.1
    conv_state = torch.randn(nb, nd, k, generator=gen) * 0.1
    x, dt, z = (torch.randn(nb, nd, generator=gen).to(bf) for _ in range(3))
    A = -torch.exp(torch.randn(nd, nn, generator=gen) * 0.5)
    Bm, Cm = torch.randn(nb, 1, nn, generator=gen).to(bf), torch.randn(nb, 1, nn, generator=gen).to(bf)
    D, bias = torch.randn(nd, generator=gen), torch.rand(nd, generator=gen) * 2 - 4
    cw = torch.rand(nd, k, generator=gen) - 0.5
    so, sg = state.clone(), state.clone().cuda()
    co, cg = conv_state.clone(), conv_state.clone().cuda()
    uo = orc.dw_causal_conv_update(co, x, cw, None, "silu")
    ug = ops.dw_causal_conv_update(cg, x.cuda(), cw.cuda(), None, "silu")
    close(ug, uo, **HALF_TOL, what="conv output")
    close(cg, co, **FP32_TOL, what="conv window")
    yo = orc.selective_state_step(so, uo, dt, A, Bm, Cm, D=D, z=z, dt_bias=bias, softplus=True)
    yg = ops.selective_state_step(sg, uo.cuda(), dt.cuda(), A.cuda(), Bm.cuda(), Cm.cuda(), D=D.cuda(), z=z.cuda(), dt_bias=bias.cuda(),
                                  softplus=True)
    close(yg, yo, **HALF_TOL, what="y")
    close(sg, so, **FP32_TOL, what="state")


def test_mamba2_decode_step_configuration_on_a_batch_slice():
    """Mamba-2 decode step at batch 256, 80 heads x 64, d_state 128 (fp32 state): the kernel at full size, batch rows
    {0, 255} against the oracle step on the flattened channels."""
    from ssm_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(6)
    kw = dict(generator=g, device="cuda")
    nb, nh, npj, nn = 256, 80, 64, 128
    bf = torch.bfloat16
    state = torch.randn(nb, nh, npj, nn, **kw) * 0.1
    x, z = torch.randn(nb, nh, npj, **kw).to(bf), torch.randn(nb, nh, npj, **kw).to(bf)
    dt = torch.randn(nb, nh, **kw).to(bf)
    A, D, bias = -torch.exp(torch.rand(nh, **kw)), torch.randn(nh, **kw), torch.randn(nh, **kw) * 0.3
    Bm, Cm = torch.randn(nb, 1, nn, **kw).to(bf), torch.randn(nb, 1, nn, **kw).to(bf)
    rows = [0, 255]
    so = state[rows].reshape(2, nh * npj, nn).cpu().clone()
    y = ops.selective_state_step_heads(state, x, dt, A, Bm, Cm, D=D, z=z, dt_bias=bias, softplus=True)
    rep = lambda v: v.cpu()[:, None].expand(nh, npj).reshape(-1)  # noqa: E731
    yo = orc.selective_state_step(so, x[rows].reshape(2, -1).cpu(), dt[rows].float().repeat_interleave(npj, dim=1).to(bf).cpu(),
                                  A.cpu()[:, None, None].expand(nh, npj, nn).reshape(nh * npj, nn), Bm[rows].cpu(), Cm[rows].cpu(),
                                  D=rep(D), z=z[rows].reshape(2, -1).cpu(), dt_bias=rep(bias), softplus=True)
    close(y[rows].reshape(2, -1), yo, **HALF_TOL, what="y")
    close(state[rows].reshape(2, nh * npj, nn), so, **FP32_TOL, what="state")


def test_initial_state_receives_a_gradient():
    from ssm_b200 import ops

    gen = torch.Generator().manual_seed(23)
    nb, nd, nl, nn = 2, 24, 75, 16
    ins = dict(u=torch.randn(nb, nd, nl, generator=gen), delta=torch.randn(nb, nd, nl, generator=gen) * 0.5,
               A=-torch.exp(torch.randn(nd, nn, generator=gen) * 0.5), B=torch.randn(nb, 1, nn, nl, generator=gen),
               C=torch.randn(nb, 1, nn, nl, generator=gen), init=torch.randn(nb, nd, nn, generator=gen))
    wy, ws = torch.randn(nb, nd, nl, generator=gen), torch.randn(nb, nd, nn, generator=gen)
    lo = {k: v.clone().requires_grad_(True) for k, v in ins.items()}
    lg = {k: v.clone().cuda().requires_grad_(True) for k, v in ins.items()}

    def manual(t):  # the oracle's scan has no initial-state argument: the same recurrence (reference.py:173-188) started from `init`
        h = t["init"]
        ys = []
        dl = F.softplus(t["delta"])
        for i in range(nl):
            h = torch.exp(dl[:, :, i, None] * t["A"][None]) * h + (dl[:, :, i] * t["u"][:, :, i])[..., None] * t["B"][:, 0, :, i][:, None, :]
            ys.append((h * t["C"][:, 0, :, i][:, None, :]).sum(-1))
        return torch.stack(ys, -1), h

    yo, so = manual(lo)
    yg, sg = ops.selective_scan(lg["u"], lg["delta"], lg["A"], lg["B"], lg["C"], softplus=True, return_last_state=True,
                                initial_state=lg["init"])
    close(yg, yo, **FP32_TOL, what="y")
    close(sg, so, **FP32_TOL, what="last state")
    go = torch.autograd.grad((yo * wy).sum() + (so * ws).sum(), list(lo.values()))
    gg = torch.autograd.grad((yg * wy.cuda()).sum() + (sg * ws.cuda()).sum(), list(lg.values()))
    for k, a, b in zip(ins, gg, go):
        close(a, b, **FP32_TOL, what=f"d{k}", reduced=k in REDUCED)


def test_in_place_edit_between_forward_and_backward_is_detected():
    from ssm_b200 import ops

    x = torch.randn(2, 8, 32, device="cuda", requires_grad=True)
    w = torch.rand(8, 4, device="cuda")
    xin = x * 1.0
    y = ops.dw_causal_conv(xin, w, None, "silu")
    xin.add_(1.0)
    with pytest.raises(RuntimeError, match="modified in place"):
        y.sum().backward()


@pytest.mark.parametrize("nb,nd,nl,dtype", [(1, 96, 2048, torch.float32), (2, 64, 1000, torch.bfloat16), (1, 32, 4096, torch.float32)])
def test_time_parallel_split_of_a_small_grid_matches_oracle(nb, nd, nl, dtype):
    """Few rows, long sequence: the forward cuts the sequence into parallel segments (local pass, serial combine, final
    pass).  Output, final state and -- through the checkpoints it writes -- every gradient must match the oracle."""
    from ssm_b200 import _lib, ops

    assert _lib.load().ssm_scan_split_segments(nb, nd, nl, 16) > 1
    gen = torch.Generator().manual_seed(nl + nd)
    ins = dict(u=torch.randn(nb, nd, nl, generator=gen).to(dtype), delta=(torch.randn(nb, nd, nl, generator=gen) - 2).to(dtype),
               A=-torch.exp(torch.randn(nd, 16, generator=gen) * 0.5), B=torch.randn(nb, 1, 16, nl, generator=gen).to(dtype),
               C=torch.randn(nb, 1, 16, nl, generator=gen).to(dtype), D=torch.randn(nd, generator=gen), z=torch.randn(nb, nd, nl, generator=gen).to(dtype),
               init=torch.randn(nb, nd, 16, generator=gen) * 0.5)
    tol = FP32_TOL if dtype == torch.float32 else HALF_TOL
    lg = {k: v.clone().cuda().requires_grad_(True) for k, v in ins.items()}
    yg, sg = ops.selective_scan(lg["u"], lg["delta"], lg["A"], lg["B"], lg["C"], D=lg["D"], z=lg["z"], softplus=True, return_last_state=True,
                                initial_state=lg["init"], keep_state_fp32=True)
    # the same recurrence (reference.py:173-188) started from `init`, in fp32 on the CPU
    f = {k: v.float() for k, v in ins.items()}
    lo = {k: v.clone().requires_grad_(True) for k, v in f.items()}
    h, ys = lo["init"], []
    dl = F.softplus(lo["delta"])
    for i in range(nl):
        h = torch.exp(dl[:, :, i, None] * lo["A"][None]) * h + (dl[:, :, i] * lo["u"][:, :, i])[..., None] * lo["B"][:, 0, :, i][:, None, :]
        ys.append((h * lo["C"][:, 0, :, i][:, None, :]).sum(-1))
    yo = (torch.stack(ys, -1) + lo["D"][None, :, None] * lo["u"]) * F.silu(lo["z"])
    close(yg, yo, **tol, what="y")
    close(sg, h, **FP32_TOL if dtype == torch.float32 else tol, what="last state")
    gen2 = torch.Generator().manual_seed(1)
    wy, ws = torch.randn(nb, nd, nl, generator=gen2).to(dtype).float(), torch.randn(nb, nd, 16, generator=gen2)  # weights the output dtype can hold
    go = torch.autograd.grad((yo * wy).sum() + (h * ws).sum(), list(lo.values()))
    gg = torch.autograd.grad((yg.float() * wy.cuda()).sum() + (sg * ws.cuda()).sum(), list(lg.values()))
    for k, a_, b_ in zip(ins, gg, go):
        close(a_, b_, **tol, what=f"d{k}", reduced=k in REDUCED)
