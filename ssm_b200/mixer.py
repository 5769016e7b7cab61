"""A Mamba-1 mixer block written against the operator surface (`ssm_b200.ops`, or any namespace
with the same five functions, e.g. the CPU oracle in tests).

Behavioural spec: the data flow of upstream's block (`src/ssm/modules/mamba1.py:176-256` for the
mixer, `src/ssm/modules/block.py:85-162` for the add + norm around it), with upstream Mamba's
parameter layout (x_proj -> dt_rank + 2 d_state, B and C shared by all channels of a token).

What is different from a line-by-line port is the activation layout: the scan-side tensors
live in ``(d_inner, B, L)`` buffers that the operators see as ``(B, d_inner, L)`` through their
row strides.  Every projection is then ONE 2-D GEMM over the ``B*L`` tokens and none of the
``permute(0, 2, 1)`` copies of the reference's forward (mamba1.py:209, 217, 226-230) exist.

`mamba1_block_forward` is the functional form (weights in a dict, operator namespace passed
in) used by the benchmark on both of its arms; `Mamba1Block` wraps it as an ``nn.Module`` with
a single-token `step` for decoding (conv-state roll + state step, reference `step`:
mamba1.py:324-385).
"""

from __future__ import annotations

import math
from typing import Any, Optional

import torch
from torch import Tensor, nn


def mamba1_mixer_forward(ops: Any, w: dict, cfg: dict, hidden: Tensor) -> Tensor:
    """The Mamba-1 mixer alone: hidden (B, L, d_model) -> (B, L, d_model), before any residual add or norm.

    ``w``: in_x, in_z (d_inner, d_model); conv_w (d_inner, K), conv_b; x_proj (R + 2N, d_inner);
    dt_proj (d_inner, R); dt_bias, A (d_inner, N), D (fp32); out_proj (d_model, d_inner).
    """
    n, r = cfg["d_state"], cfg["dt_rank"]
    nb, nl, dm = hidden.shape
    di = w["in_x"].shape[0]
    h2 = hidden.reshape(nb * nl, dm)

    def rows(m2d):  # (C, B*L) -> (B, C, L) view
        return m2d.view(m2d.shape[0], nb, nl).permute(1, 0, 2)

    x = rows(torch.matmul(w["in_x"], h2.t()))
    z = rows(torch.matmul(w["in_z"], h2.t()))
    u = ops.dw_causal_conv(x, w["conv_w"], w["conv_b"], "silu")
    u2 = u.permute(1, 0, 2).reshape(di, nb * nl)                       # (Di, B*L), no copy for the channel-major layout
    x_dbl = torch.matmul(w["x_proj"], u2)                              # (R + 2N, B*L)
    dt_low, Bm, Cm = torch.split(x_dbl, [r, n, n], dim=0)
    delta = rows(torch.matmul(w["dt_proj"], dt_low))                   # (B, Di, L) view
    Bg = Bm.view(n, nb, nl).permute(1, 0, 2).unsqueeze(1)              # (B, 1, N, L)
    Cg = Cm.view(n, nb, nl).permute(1, 0, 2).unsqueeze(1)
    y = ops.selective_scan(u, delta, w["A"], Bg, Cg, D=w["D"], z=z, dt_bias=w["dt_bias"], softplus=True)
    y2 = y.permute(1, 0, 2).reshape(di, nb * nl)
    return torch.matmul(y2.t(), w["out_proj"].t()).view(nb, nl, dm)     # (B, L, d_model)


def mamba1_block_forward(ops: Any, w: dict, cfg: dict, hidden: Tensor, residual: Optional[Tensor]):
    """hidden (B, L, d_model) activations, residual (B, L, d_model) fp32 stream or None
    -> (normed, new_residual): new_residual = residual + mixer(hidden); normed = RMSNorm(new_residual).

    ``w``: the mixer weights of :func:`mamba1_mixer_forward` plus norm_w.
    """
    out = mamba1_mixer_forward(ops, w, cfg, hidden)
    return ops.fused_layer_norm(out, w["norm_w"], None, residual=residual, is_rms=True, eps=cfg.get("eps", 1e-5), prenorm=True,
                                residual_in_fp32=True, return_residual=True)


def mamba1_mixer_step(ops: Any, w: dict, cfg: dict, tok: Tensor, conv_state: Tensor, ssm_state: Tensor) -> Tensor:
    """One decode token through the Mamba-1 mixer: tok (B, d_model) -> (B, d_model); ``conv_state (B, d_inner, K)`` and
    ``ssm_state (B, d_inner, N)`` (both fp32) are updated in place (reference step: modules/mamba1.py:324-385)."""
    n, r = cfg["d_state"], cfg["dt_rank"]
    x, z = tok @ w["in_x"].t(), tok @ w["in_z"].t()
    u = ops.dw_causal_conv_update(conv_state, x, w["conv_w"], w["conv_b"], "silu")
    xd = u @ w["x_proj"].t()
    delta = xd[:, :r] @ w["dt_proj"].t()
    y = ops.selective_state_step(ssm_state, u, delta, w["A"], xd[:, r:r + n].unsqueeze(1), xd[:, r + n:].unsqueeze(1),
                                 D=w["D"], z=z, dt_bias=w["dt_bias"], softplus=True)
    return y @ w["out_proj"].t()


class Mamba1Block(nn.Module):
    """Mixer + residual add + RMSNorm on the five operators.  ``forward(hidden, residual)`` returns
    ``(normed, residual)`` like the reference's fused-add-norm block; ``step`` advances one token."""

    def __init__(self, d_model: int, d_state: int = 16, d_conv: int = 4, expand: int = 2, dt_rank: int | str = "auto",
                 dt_min: float = 1e-3, dt_max: float = 1e-1, dt_init_floor: float = 1e-4, eps: float = 1e-5,
                 device=None, dtype=None, ops: Any = None) -> None:
        super().__init__()
        if isinstance(dt_rank, str):
            if dt_rank != "auto":
                raise ValueError("dt_rank must be an integer or 'auto'.")
            dt_rank = math.ceil(d_model / 16)
        if dt_rank <= 0:
            raise ValueError("dt_rank must be positive when provided as an integer.")
        if dt_min <= 0 or dt_max <= 0 or dt_min > dt_max:
            raise ValueError("dt_min and dt_max must be positive with dt_min <= dt_max.")
        self.d_model, self.d_state, self.d_conv, self.dt_rank = d_model, d_state, d_conv, int(dt_rank)
        self.d_inner = expand * d_model
        self.eps = eps
        self._ops = ops
        kw = dict(device=device, dtype=dtype)
        f32 = dict(device=device, dtype=torch.float32)
        di, r, n = self.d_inner, self.dt_rank, d_state

        def lin(o, i):
            return nn.Parameter(torch.randn(o, i, **kw) / i ** 0.5)

        self.in_x, self.in_z = lin(di, d_model), lin(di, d_model)
        self.conv_w = nn.Parameter((torch.rand(di, d_conv, **kw) - 0.5) * (2.0 / d_conv ** 0.5))
        self.conv_b = nn.Parameter(torch.zeros(di, **kw))
        self.x_proj = lin(r + 2 * n, di)
        self.dt_proj = nn.Parameter((torch.rand(di, r, **kw) * 2 - 1) * r ** -0.5)
        dt = torch.exp(torch.rand(di, **f32) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=dt_init_floor)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))  # inverse softplus of the sampled step
        self.A_log = nn.Parameter(torch.log(torch.arange(1, n + 1, **f32)).repeat(di, 1))
        self.D = nn.Parameter(torch.ones(di, **f32))
        self.out_proj = lin(d_model, di)
        self.norm_w = nn.Parameter(torch.ones(d_model, **kw))

    def _namespace(self):
        if self._ops is not None:
            return self._ops
        from . import ops  # the CUDA operators; raises if the library has not been built

        return ops

    def _weights(self) -> dict:
        return dict(in_x=self.in_x, in_z=self.in_z, conv_w=self.conv_w, conv_b=self.conv_b, x_proj=self.x_proj, dt_proj=self.dt_proj,
                    dt_bias=self.dt_bias, A=-torch.exp(self.A_log), D=self.D, out_proj=self.out_proj, norm_w=self.norm_w)

    def forward(self, hidden: Tensor, residual: Optional[Tensor] = None):
        if hidden.ndim != 3 or hidden.shape[-1] != self.d_model:
            raise ValueError("hidden_states must have shape (B, L, d_model).")
        cfg = dict(d_state=self.d_state, dt_rank=self.dt_rank, eps=self.eps)
        return mamba1_block_forward(self._namespace(), self._weights(), cfg, hidden, residual)

    def mixer_forward(self, u: Tensor) -> Tensor:
        """The mixer alone (no residual add, no norm): u (B, L, d_model) -> (B, L, d_model)."""
        return mamba1_mixer_forward(self._namespace(), self._weights(), dict(d_state=self.d_state, dt_rank=self.dt_rank), u)

    def mixer_step(self, tok: Tensor, cache) -> Tensor:
        """The mixer alone on one token: tok (B, d_model) -> (B, d_model); ``cache`` from `allocate_inference_cache`."""
        return mamba1_mixer_step(self._namespace(), self._weights(), dict(d_state=self.d_state, dt_rank=self.dt_rank), tok, cache[0], cache[1])

    def allocate_inference_cache(self, batch_size: int, dtype: Optional[torch.dtype] = None):
        """(conv_state (B, d_inner, K), ssm_state (B, d_inner, N)), both fp32 and zero-filled."""
        del dtype  # both states are kept in fp32 whatever the activation dtype
        dev = self.in_x.device
        return (torch.zeros(batch_size, self.d_inner, self.d_conv, device=dev, dtype=torch.float32),
                torch.zeros(batch_size, self.d_inner, self.d_state, device=dev, dtype=torch.float32))

    def step(self, hidden: Tensor, residual: Optional[Tensor], conv_state: Tensor, ssm_state: Tensor):
        """One token: hidden (B, 1, d_model) -> (normed (B, 1, d_model), new residual); both states are updated in place."""
        if hidden.ndim != 3 or hidden.shape[1] != 1:
            raise ValueError("step expects inputs of shape (B, 1, d_model)")
        ops = self._namespace()
        cfg = dict(d_state=self.d_state, dt_rank=self.dt_rank)
        out = mamba1_mixer_step(ops, self._weights(), cfg, hidden[:, 0], conv_state, ssm_state).unsqueeze(1)
        res1 = None if residual is None else residual
        return ops.fused_layer_norm(out, self.norm_w, None, residual=res1, is_rms=True, eps=self.eps, prenorm=True,
                                    residual_in_fp32=True, return_residual=True)


def mamba2_block_forward(ops: Any, w: dict, cfg: dict, hidden: Tensor, residual: Optional[Tensor], group=None, sharded: bool = False):
    """One Mamba-2 block (upstream Mamba-2 data flow; the reference's ``Mamba2`` has no ``d_state`` axis, so the
    layout follows upstream): ``residual += hidden; u = RMSNorm(residual); out = mixer(u)`` -> ``(out, residual)``.

    mixer: projections of u to z, x, B, C, dt (separate GEMMs, so every operand of the scan is contiguous);
    depthwise causal conv + SiLU on x, B and C (channels-last); SSD scan with D skip, dt bias + softplus and
    the SiLU(z) gate; RMSNorm over d_inner; out projection.

    ``sharded=True``: ``hidden`` is this rank's contiguous shard of the sequence; the conv inputs of the last
    K-1 tokens go to the next rank and the chunk state is handed over (`ssm_b200.seqpar`), CUDA operators only.
    ``cfg``: heads, headdim, d_state, groups, chunk_size, eps.
    """
    eps = cfg.get("eps", 1e-5)
    u, residual = ops.fused_layer_norm(hidden, w["pre_norm_w"], None, residual=residual, is_rms=True, eps=eps, prenorm=True,
                                       residual_in_fp32=True, return_residual=True)
    return mamba2_mixer_forward(ops, w, cfg, u, group=group, sharded=sharded), residual


def mamba2_mixer_forward(ops: Any, w: dict, cfg: dict, u: Tensor, group=None, sharded: bool = False) -> Tensor:
    """The Mamba-2 mixer alone on normed activations u (B, L, d_model) -> (B, L, d_model); see `mamba2_block_forward`."""
    nb, nl, dm = u.shape
    nh, hp, n, g = cfg["heads"], cfg["headdim"], cfg["d_state"], cfg["groups"]
    eps = cfg.get("eps", 1e-5)
    u2 = u.reshape(nb * nl, dm)

    def proj(name):
        return torch.matmul(u2, w[name].t()).view(nb, nl, -1)

    px, pB, pC = proj("in_x"), proj("in_B"), proj("in_C")
    halos = [None, None, None]
    if sharded:
        from . import seqpar

        # one message for the three inputs; the step-size projection is enqueued while it travels
        posted = seqpar.post_conv_halos([px, pB, pC], w["conv_x"].shape[1], group)
        dt = proj("in_dt")
        halos = posted.wait()

    def conv(t, name, halo):
        if halo is None:
            return ops.dw_causal_conv(t, w[name], w[name + "_b"], "silu")
        return ops.dw_causal_conv(t, w[name], w[name + "_b"], "silu", halo=halo)

    x = conv(px, "conv_x", halos[0]).view(nb, nl, nh, hp)
    Bm = conv(pB, "conv_B", halos[1]).view(nb, nl, g, n)
    Cm = conv(pC, "conv_C", halos[2]).view(nb, nl, g, n)
    A = -torch.exp(w["A_log"])
    if sharded:
        from . import seqpar

        # the gate's projection is the largest piece of work that does not depend on the other shards: it is enqueued after
        # this shard's state phase, while the states are gathered and the ranks wait for the slowest of them
        y, _ = seqpar.ssd_scan_sharded(x, dt, A, Bm, Cm, cfg.get("chunk_size", 256), D=w["D"], z=lambda: proj("in_z").view(nb, nl, nh, hp),
                                       dt_bias=w["dt_bias"], dt_softplus=True, group=group)
    else:
        z = proj("in_z").view(nb, nl, nh, hp)
        dt = proj("in_dt")
        y = ops.ssd_scan(x, dt, A, Bm, Cm, cfg.get("chunk_size", 256), D=w["D"], z=z, dt_bias=w["dt_bias"], dt_softplus=True)
    y = ops.fused_layer_norm(y.reshape(nb, nl, nh * hp), w["norm_w"], None, is_rms=True, eps=eps)
    return torch.matmul(y.reshape(nb * nl, nh * hp), w["out_proj"].t()).view(nb, nl, dm)


def mamba2_mixer_step(ops: Any, w: dict, cfg: dict, tok: Tensor, conv_states: tuple, ssm_state: Tensor) -> Tensor:
    """One decode token through the Mamba-2 mixer: tok (B, d_model), normed -> (B, d_model).  ``conv_states``: the rolling
    windows of the x, B and C convolutions ((B, C_i, K) fp32 each); ``ssm_state (B, H, P, N)`` fp32; all updated in place."""
    nb = tok.shape[0]
    nh, hp, n, g = cfg["heads"], cfg["headdim"], cfg["d_state"], cfg["groups"]
    eps = cfg.get("eps", 1e-5)
    z = tok @ w["in_z"].t()
    x = ops.dw_causal_conv_update(conv_states[0], tok @ w["in_x"].t(), w["conv_x"], w["conv_x_b"], "silu")
    Bm = ops.dw_causal_conv_update(conv_states[1], tok @ w["in_B"].t(), w["conv_B"], w["conv_B_b"], "silu").view(nb, g, n)
    Cm = ops.dw_causal_conv_update(conv_states[2], tok @ w["in_C"].t(), w["conv_C"], w["conv_C_b"], "silu").view(nb, g, n)
    dt = tok @ w["in_dt"].t()
    A = -torch.exp(w["A_log"])
    if hasattr(ops, "selective_state_step_heads"):
        y = ops.selective_state_step_heads(ssm_state, x.view(nb, nh, hp), dt, A, Bm, Cm, D=w["D"], z=z.view(nb, nh, hp),
                                           dt_bias=w["dt_bias"], softplus=True).reshape(nb, nh * hp)
    else:  # operator namespaces without the per-head form (the CPU oracle): the same step on the flattened channels
        flat = ssm_state.view(nb, nh * hp, n)
        rep = lambda v: v[:, None].expand(nh, hp).reshape(-1)  # noqa: E731
        y = ops.selective_state_step(flat, x, dt.repeat_interleave(hp, dim=1), A[:, None, None].expand(nh, hp, n).reshape(nh * hp, n), Bm, Cm,
                                     D=rep(w["D"]), z=z, dt_bias=rep(w["dt_bias"]), softplus=True)
    y = ops.fused_layer_norm(y.view(nb, 1, nh * hp), w["norm_w"], None, is_rms=True, eps=eps)
    return y.view(nb, nh * hp) @ w["out_proj"].t()


class Mamba2Block(nn.Module):
    """Pre-norm Mamba-2 block on the operators: ``forward(hidden, residual) -> (mixer output, residual stream)``.
    ``forward(..., sharded=True, group=pg)`` runs it on one contiguous shard of a sequence split over ranks."""

    def __init__(self, d_model: int, d_state: int = 128, d_conv: int = 4, expand: int = 2, headdim: int = 64, ngroups: int = 1,
                 chunk_size: int = 256, dt_min: float = 1e-3, dt_max: float = 1e-1, dt_init_floor: float = 1e-4, eps: float = 1e-5,
                 device=None, dtype=None, ops: Any = None) -> None:
        super().__init__()
        d_inner = expand * d_model
        if d_inner % headdim:
            raise ValueError("expand * d_model must be a multiple of headdim.")
        heads = d_inner // headdim
        if heads % ngroups:
            raise ValueError("Group dimension must divide H.")
        self.d_model, self.d_inner, self.d_state, self.d_conv = d_model, d_inner, d_state, d_conv
        self.heads, self.headdim, self.ngroups, self.chunk_size, self.eps = heads, headdim, ngroups, chunk_size, eps
        self._ops = ops
        kw = dict(device=device, dtype=dtype)
        f32 = dict(device=device, dtype=torch.float32)
        gn = ngroups * d_state

        def lin(o, i):
            return nn.Parameter(torch.randn(o, i, **kw) / i ** 0.5)

        def conv_w(c):
            return nn.Parameter((torch.rand(c, d_conv, **kw) - 0.5) * (2.0 / d_conv ** 0.5))

        self.pre_norm_w = nn.Parameter(torch.ones(d_model, **kw))
        self.in_z, self.in_x, self.in_B, self.in_C, self.in_dt = lin(d_inner, d_model), lin(d_inner, d_model), lin(gn, d_model), lin(gn, d_model), lin(heads, d_model)
        self.conv_x, self.conv_B, self.conv_C = conv_w(d_inner), conv_w(gn), conv_w(gn)
        self.conv_x_b, self.conv_B_b, self.conv_C_b = (nn.Parameter(torch.zeros(c, **kw)) for c in (d_inner, gn, gn))
        dt = torch.exp(torch.rand(heads, **f32) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=dt_init_floor)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        self.A_log = nn.Parameter(torch.log(torch.empty(heads, **f32).uniform_(1.0, 16.0)))
        self.D = nn.Parameter(torch.ones(heads, **f32))
        self.norm_w = nn.Parameter(torch.ones(d_inner, **kw))
        self.out_proj = lin(d_model, d_inner)

    def _namespace(self):
        if self._ops is not None:
            return self._ops
        from . import ops  # the CUDA operators; raises if the library has not been built

        return ops

    def _cfg(self) -> dict:
        return dict(heads=self.heads, headdim=self.headdim, d_state=self.d_state, groups=self.ngroups, chunk_size=self.chunk_size, eps=self.eps)

    def forward(self, hidden: Tensor, residual: Optional[Tensor] = None, sharded: bool = False, group=None):
        if hidden.ndim != 3 or hidden.shape[-1] != self.d_model:
            raise ValueError("hidden_states must have shape (B, L, d_model).")
        w = {k: v for k, v in self.named_parameters()}
        return mamba2_block_forward(self._namespace(), w, self._cfg(), hidden, residual, group=group, sharded=sharded)

    def mixer_forward(self, u: Tensor, sharded: bool = False, group=None) -> Tensor:
        """The mixer alone on normed activations: u (B, L, d_model) -> (B, L, d_model)."""
        return mamba2_mixer_forward(self._namespace(), {k: v for k, v in self.named_parameters()}, self._cfg(), u, group=group, sharded=sharded)

    def allocate_inference_cache(self, batch_size: int, dtype: Optional[torch.dtype] = None):
        """((conv windows of x, B, C: (B, C_i, K)), ssm_state (B, H, P, N)), all fp32 and zero-filled."""
        del dtype
        dev = self.in_x.device
        gn = self.ngroups * self.d_state
        z = lambda c: torch.zeros(batch_size, c, self.d_conv, device=dev, dtype=torch.float32)  # noqa: E731
        return ((z(self.d_inner), z(gn), z(gn)), torch.zeros(batch_size, self.heads, self.headdim, self.d_state, device=dev, dtype=torch.float32))

    def mixer_step(self, tok: Tensor, cache) -> Tensor:
        """The mixer alone on one normed token: tok (B, d_model) -> (B, d_model); ``cache`` from `allocate_inference_cache`."""
        return mamba2_mixer_step(self._namespace(), {k: v for k, v in self.named_parameters()}, self._cfg(), tok, cache[0], cache[1])
