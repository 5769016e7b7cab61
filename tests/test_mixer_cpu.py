"""The Mamba-1 block of `ssm_b200.mixer` on the CPU oracle: its channel-major data flow must equal a
plain batch-major restatement of the same block, and its one-token `step` must reproduce `forward`."""

from __future__ import annotations

import torch

from oracle import ssm_oracle as orc
from ssm_b200.mixer import Mamba1Block


def _batch_major_block(m: Mamba1Block, hidden, residual):
    """The same block with (B, L, C) linears and explicit permutes, as the reference's modules are written."""
    nb, nl, _ = hidden.shape
    x = hidden @ m.in_x.t()
    z = hidden @ m.in_z.t()
    u = orc.dw_causal_conv(x.permute(0, 2, 1), m.conv_w, m.conv_b, "silu")               # (B, Di, L)
    xd = u.permute(0, 2, 1) @ m.x_proj.t()
    r, n = m.dt_rank, m.d_state
    delta = (xd[..., :r] @ m.dt_proj.t()).permute(0, 2, 1)
    Bm = xd[..., r:r + n].permute(0, 2, 1).unsqueeze(1)
    Cm = xd[..., r + n:].permute(0, 2, 1).unsqueeze(1)
    y = orc.selective_scan(u, delta, -torch.exp(m.A_log), Bm, Cm, D=m.D, z=z.permute(0, 2, 1), dt_bias=m.dt_bias, softplus=True)
    out = y.permute(0, 2, 1) @ m.out_proj.t()
    return orc.fused_layer_norm(out, m.norm_w, None, residual=residual, is_rms=True, eps=m.eps, prenorm=True, residual_in_fp32=True,
                                return_residual=True)


def test_block_matches_batch_major_restatement_and_has_gradients():
    torch.manual_seed(0)
    m = Mamba1Block(32, d_state=8, d_conv=4, expand=2, ops=orc)
    hidden = torch.randn(2, 19, 32, requires_grad=True)
    residual = torch.randn(2, 19, 32)
    y1, r1 = m(hidden, residual)
    y2, r2 = _batch_major_block(m, hidden, residual)
    torch.testing.assert_close(y1, y2, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(r1, r2, rtol=1e-5, atol=1e-6)
    g1 = torch.autograd.grad(y1.square().sum(), [hidden, m.x_proj, m.A_log], retain_graph=True)
    g2 = torch.autograd.grad(y2.square().sum(), [hidden, m.x_proj, m.A_log])
    for a, b in zip(g1, g2):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


def test_step_reproduces_forward_token_by_token():
    torch.manual_seed(1)
    m = Mamba1Block(24, d_state=4, d_conv=3, expand=2, ops=orc)
    hidden = torch.randn(3, 7, 24)
    residual = torch.randn(3, 7, 24)
    with torch.no_grad():
        y, r = m(hidden, residual)
        conv_state, ssm_state = m.allocate_inference_cache(3)
        for t in range(7):
            yt, rt = m.step(hidden[:, t:t + 1], residual[:, t:t + 1], conv_state, ssm_state)
            torch.testing.assert_close(yt, y[:, t:t + 1], rtol=1e-5, atol=1e-6)
            torch.testing.assert_close(rt, r[:, t:t + 1], rtol=1e-5, atol=1e-6)


def test_constructor_rejects_bad_arguments():
    import pytest

    with pytest.raises(ValueError):
        Mamba1Block(16, dt_rank="big", ops=orc)
    with pytest.raises(ValueError):
        Mamba1Block(16, dt_rank=0, ops=orc)
    with pytest.raises(ValueError):
        Mamba1Block(16, dt_min=0.2, dt_max=0.1, ops=orc)
    with pytest.raises(ValueError):
        Mamba1Block(16, ops=orc)(torch.zeros(2, 16))


def test_mamba2_block_runs_on_the_oracle_and_matches_a_token_loop():
    """Mamba-2 block on the CPU oracle against a direct per-token recurrence of the same block."""
    from ssm_b200.mixer import Mamba2Block

    torch.manual_seed(2)
    m = Mamba2Block(16, d_state=8, d_conv=3, expand=2, headdim=8, ngroups=2, chunk_size=4, ops=orc)
    hidden = torch.randn(2, 11, 16)
    residual = torch.randn(2, 11, 16)
    with torch.no_grad():
        out, res = m(hidden, residual)
        # restatement: explicit recurrence h_t = exp(dt A) h + dt B x^T per head
        r = hidden + residual
        u = r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + m.eps) * m.pre_norm_w

        def conv(t, wgt, b):
            k = wgt.shape[1]
            tp = torch.nn.functional.pad(t.transpose(1, 2), (k - 1, 0))
            return torch.nn.functional.silu(torch.nn.functional.conv1d(tp, wgt.unsqueeze(1), b, groups=wgt.shape[0])).transpose(1, 2)

        z = (u @ m.in_z.t()).view(2, 11, m.heads, m.headdim)
        x = conv(u @ m.in_x.t(), m.conv_x, m.conv_x_b).view(2, 11, m.heads, m.headdim)
        Bm = conv(u @ m.in_B.t(), m.conv_B, m.conv_B_b).view(2, 11, m.ngroups, m.d_state)
        Cm = conv(u @ m.in_C.t(), m.conv_C, m.conv_C_b).view(2, 11, m.ngroups, m.d_state)
        dt = torch.nn.functional.softplus(u @ m.in_dt.t() + m.dt_bias)
        A = -torch.exp(m.A_log)
        hpg = m.heads // m.ngroups
        state = torch.zeros(2, m.heads, m.headdim, m.d_state)
        ys = []
        for t in range(11):
            Bt = Bm[:, t].repeat_interleave(hpg, dim=1)
            Ct = Cm[:, t].repeat_interleave(hpg, dim=1)
            decay = torch.exp(dt[:, t] * A)[:, :, None, None]
            state = decay * state + dt[:, t][:, :, None, None] * x[:, t][..., None] * Bt[:, :, None, :]
            y = (state * Ct[:, :, None, :]).sum(-1) + m.D[None, :, None] * x[:, t]
            ys.append(y * torch.nn.functional.silu(z[:, t]))
        y = torch.stack(ys, dim=1).reshape(2, 11, m.d_inner)
        y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + m.eps) * m.norm_w
        ref = y @ m.out_proj.t()
    torch.testing.assert_close(res, r, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
