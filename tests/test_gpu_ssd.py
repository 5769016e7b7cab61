"""The tcgen05 state-space-dual kernels against the CPU oracle (and against the scan-kernel
path of the same operator) at shapes the tensor-core path is built for."""

from __future__ import annotations

import pytest
import torch

from oracle import ssm_oracle as orc
from tests.gpu_util import FP32_TOL, HALF_TOL, close

pytestmark = pytest.mark.gpu

# every output element of the tensor-core path is a 256-term product sum of bf16-rounded operands
SSD_TOL = dict(rtol=2e-2, atol=2e-2)


def _inputs(nb, nl, nh, ng, dtype, seed, with_init=True):
    gen = torch.Generator().manual_seed(seed)
    npj, nn = 64, 128
    X = torch.randn(nb, nl, nh, npj, generator=gen).to(dtype)
    dt = (torch.randn(nb, nl, nh, generator=gen) - 3.0).to(dtype)
    A = -torch.exp(torch.rand(nh, generator=gen) * 2.77)
    Bm = (torch.randn(nb, nl, ng, nn, generator=gen) / nn ** 0.5).to(dtype)
    Cm = (torch.randn(nb, nl, ng, nn, generator=gen) / nn ** 0.5).to(dtype)
    D = torch.randn(nh, generator=gen)
    z = torch.randn(nb, nl, nh, npj, generator=gen).to(dtype)
    bias = torch.randn(nh, generator=gen) * 0.3
    init = torch.randn(nb, nh, npj, nn, generator=gen) * 0.5 if with_init else None
    return dict(X=X, dt=dt, A=A, B=Bm, C=Cm, D=D, z=z, dt_bias=bias, initial_states=init)


CASES = [
    # batch, len, heads, groups, dtype
    (1, 256, 1, 1, torch.bfloat16),
    (2, 512, 3, 1, torch.bfloat16),
    (1, 700, 4, 2, torch.bfloat16),   # ragged last chunk, two groups
    (1, 512, 2, 1, torch.float16),
    (1, 100, 2, 2, torch.bfloat16),   # shorter than one row block
    (2, 300, 96, 2, torch.bfloat16),  # more (batch, head) pairs than SMs: two heads per state CTA
    (3, 256, 120, 1, torch.float16),  # three heads per state CTA
    (5, 256, 128, 1, torch.bfloat16),  # four heads per state CTA
]


@pytest.mark.parametrize("nb,nl,nh,ng,dtype", CASES)
def test_tensor_core_ssd_matches_oracle(nb, nl, nh, ng, dtype):
    from ssm_b200 import ops

    t = _inputs(nb, nl, nh, ng, dtype, seed=nl + nh)
    assert ops.ssd_tensor_core_supported(t["X"].cuda(), t["B"].cuda(), 256)
    Yo, So = orc.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 256, D=t["D"], z=t["z"], dt_bias=t["dt_bias"], dt_softplus=True,
                          initial_states=t["initial_states"], return_final_states=True)
    g = {k: (None if v is None else v.cuda()) for k, v in t.items()}
    Yg, Sg = ops.ssd_scan(g["X"], g["dt"], g["A"], g["B"], g["C"], 256, D=g["D"], z=g["z"], dt_bias=g["dt_bias"], dt_softplus=True,
                          initial_states=g["initial_states"], return_final_states=True, check_status=True)
    assert Yg.dtype == dtype and Sg.dtype == torch.float32
    close(Yg, Yo, **SSD_TOL, what="Y", reduced=True)
    close(Sg, So, **SSD_TOL, what="final state", reduced=True)


def test_tensor_core_ssd_without_optionals_and_matrix_D():
    from ssm_b200 import ops

    t = _inputs(1, 512, 2, 1, torch.bfloat16, seed=9, with_init=False)
    Dm = torch.randn(2, 64)
    dtp = (t["dt"].float().abs() * 0.05 + 0.01).to(torch.bfloat16)
    Yo, So = orc.ssd_scan(t["X"], dtp, t["A"], t["B"], t["C"], 256, D=Dm, return_final_states=True)
    Yg, Sg = ops.ssd_scan(t["X"].cuda(), dtp.cuda(), t["A"].cuda(), t["B"].cuda(), t["C"].cuda(), 256, D=Dm.cuda(),
                          return_final_states=True, check_status=True)
    close(Yg, Yo, **SSD_TOL, what="Y", reduced=True)
    close(Sg, So, **SSD_TOL, what="final state", reduced=True)


def test_tensor_core_ssd_strong_decay_takes_the_exact_mask_form():
    """Steps whose decay inside a 32-step chunk exceeds 2^60 cannot use the factored mask; mixed with mild heads."""
    from ssm_b200 import ops

    t = _inputs(1, 768, 4, 1, torch.bfloat16, seed=21)
    A = torch.tensor([-16.0, -0.5, -12.0, -1.0])
    dtp = torch.rand(1, 768, 4, generator=torch.Generator().manual_seed(5)).mul(0.6).add(0.05).to(torch.bfloat16)
    dtp[:, 300:340] = 0.0  # steps without any update
    Yo, So = orc.ssd_scan(t["X"], dtp, A, t["B"], t["C"], 256, D=t["D"], z=t["z"], initial_states=t["initial_states"], return_final_states=True)
    Yg, Sg = ops.ssd_scan(t["X"].cuda(), dtp.cuda(), A.cuda(), t["B"].cuda(), t["C"].cuda(), 256, D=t["D"].cuda(), z=t["z"].cuda(),
                          initial_states=t["initial_states"].cuda(), return_final_states=True, check_status=True)
    assert torch.isfinite(Yg.float()).all() and torch.isfinite(Sg).all()
    close(Yg, Yo, **SSD_TOL, what="Y", reduced=True)
    close(Sg, So, **SSD_TOL, what="final state", reduced=True)


def test_tensor_core_ssd_agrees_with_scan_kernel_path_and_has_gradients():
    """Same operator, two CUDA paths: chunked tensor-core GEMMs vs the sequential scan kernels."""
    from ssm_b200 import ops

    t = {k: (None if v is None else v.cuda()) for k, v in _inputs(2, 768, 4, 1, torch.bfloat16, seed=4).items()}
    Y1, S1 = ops.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 256, D=t["D"], z=t["z"], dt_bias=t["dt_bias"], dt_softplus=True,
                          initial_states=t["initial_states"], return_final_states=True, check_status=True)
    Y2, S2 = ops._ssd_via_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], t["D"], t["z"], t["dt_bias"], True, t["initial_states"])
    close(Y1, Y2, **SSD_TOL, what="Y", reduced=True)
    close(S1, S2, **SSD_TOL, what="final state", reduced=True)
    # chaining: second half started from the first half's final state
    h = 512
    Ya, Sa = ops.ssd_scan(t["X"][:, :h], t["dt"][:, :h], t["A"], t["B"][:, :h], t["C"][:, :h], 256, D=t["D"], z=t["z"][:, :h],
                          dt_bias=t["dt_bias"], dt_softplus=True, initial_states=t["initial_states"], return_final_states=True)
    Yb, Sb = ops.ssd_scan(t["X"][:, h:], t["dt"][:, h:], t["A"], t["B"][:, h:], t["C"][:, h:], 256, D=t["D"], z=t["z"][:, h:],
                          dt_bias=t["dt_bias"], dt_softplus=True, initial_states=Sa, return_final_states=True)
    close(torch.cat([Ya, Yb], 1), Y1, **SSD_TOL, what="chained Y", reduced=True)
    close(Sb, S1, **SSD_TOL, what="chained state", reduced=True)
    # gradients flow (through the scan-kernel backward)
    X = t["X"].clone().requires_grad_(True)
    A = t["A"].clone().requires_grad_(True)
    Y = ops.ssd_scan(X, t["dt"], A, t["B"], t["C"], 256, dt_softplus=True)
    Y.float().square().mean().backward()
    assert X.grad is not None and torch.isfinite(X.grad.float()).all() and float(X.grad.float().abs().max()) > 0
    assert A.grad is not None and torch.isfinite(A.grad).all()


def test_two_phase_shards_reproduce_the_unsharded_scan():
    """The state phase / finish phase split that sequence sharding uses, with two shards emulated on
    one GPU: shard states folded on the host side must give the unsharded result."""
    from ssm_b200 import ops, seqpar

    t = {k: (None if v is None else v.cuda()) for k, v in _inputs(2, 1024, 3, 1, torch.bfloat16, seed=21).items()}
    Yf, Sf = ops.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 256, D=t["D"], z=t["z"], dt_bias=t["dt_bias"], dt_softplus=True,
                          initial_states=t["initial_states"], return_final_states=True)
    h = 512
    shards = []
    for sl in (slice(0, h), slice(h, 1024)):
        w = ops._SsdWorkspace(t["X"][:, sl], t["dt"][:, sl], t["A"], t["B"][:, sl], t["C"][:, sl], t["D"], t["z"][:, sl], t["dt_bias"], True, 256)
        _, s_loc = w.run(1, None, False)
        shards.append((w, s_loc, w.total_log_decay()))
    states, logp = [s[1] for s in shards], [s[2] for s in shards]
    ref_logp = (torch.nn.functional.softplus(t["dt"][:, :h].float() + t["dt_bias"]) * t["A"]).sum(1)
    close(logp[0], ref_logp, rtol=1e-3, atol=1e-3, what="shard log-decay")
    outs = []
    for r, (w, _, _) in enumerate(shards):
        s_in = seqpar.fold_incoming_state(states, logp, r, t["initial_states"])
        outs.append(w.run(2, s_in, True))
    close(torch.cat([outs[0][0], outs[1][0]], 1), Yf, **SSD_TOL, what="Y", reduced=True)
    close(outs[1][1], Sf, **SSD_TOL, what="final state", reduced=True)
    assert int(shards[0][0].status.item()) == 0 and int(shards[1][0].status.item()) == 0


def test_shard_summary_and_fold_kernel_match_the_host_fold():
    """Phase 1 leaves (final state | total log-decay) in the scratch; the fold entry point turns the gathered
    summaries of all ranks into a rank's incoming state exactly like the host-side fold."""
    from ssm_b200 import _lib as L
    from ssm_b200 import ops, seqpar

    world, nb, nh = 3, 2, 3
    summaries, states, logps = [], [], []
    for r in range(world):
        t = {k: (None if v is None else v.cuda()) for k, v in _inputs(nb, 512, nh, 1, torch.bfloat16, seed=40 + r, with_init=False).items()}
        w = ops._SsdWorkspace(t["X"], t["dt"], t["A"], t["B"], t["C"], t["D"], t["z"], t["dt_bias"], True, 256)
        _, s_loc = w.run(1, None, False)
        summary = w.shard_summary().clone()
        assert summary.numel() == L.load().ssm_ssd_shard_summary_floats(nb, nh)
        close(summary[: s_loc.numel()].view_as(s_loc), s_loc, **FP32_TOL, what="state part of the summary")
        close(summary[s_loc.numel():].view(nb, nh), w.total_log_decay(), **FP32_TOL, what="log-decay part of the summary")
        summaries.append(summary), states.append(s_loc), logps.append(w.total_log_decay())
    gathered = torch.cat(summaries)
    init = torch.randn(nb, nh, 64, 128, device="cuda")
    for r in range(world):
        for ini in (None, init):
            out = torch.empty(nb, nh, 64, 128, device="cuda")
            L.check(L.load().ssm_ssd_fold_shards(gathered.data_ptr(), world, r, nb, nh, None if ini is None else ini.data_ptr(), out.data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream))
            close(out, seqpar.fold_incoming_state(states, logps, r, ini), **FP32_TOL, what=f"incoming state of rank {r}")


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """The library's self-test makes a bounded device wait run out (a barrier nothing arms, 100 probes).  The status word is
    reported without a synchronisation by the next call, or at once by `ssd_check_status`; afterwards the same operator runs
    and matches the oracle again."""
    from ssm_b200 import ops

    t = {k: (None if v is None else v.cuda()) for k, v in _inputs(1, 256, 2, 1, torch.bfloat16, seed=3, with_init=False).items()}
    ops.ssd_check_status()  # clean before
    ops.ssd_wait_selftest(100)
    with pytest.raises(RuntimeError, match="bounded device-side wait ran out"):
        ops.ssd_check_status()
    ops.ssd_check_status()  # the report cleared the word
    # the lazy path: the next operator call surfaces an earlier failure without synchronising for it
    ops.ssd_wait_selftest(100)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status 3"):
        ops.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 256, dt_softplus=True)
    Yg = ops.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 256, dt_softplus=True, check_status=True)
    Yo = orc.ssd_scan(t["X"].cpu(), t["dt"].cpu(), t["A"].cpu(), t["B"].cpu(), t["C"].cpu(), 256, dt_softplus=True)
    close(Yg, Yo, **SSD_TOL, what="Y after the reported failure", reduced=True)
