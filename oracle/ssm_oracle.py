"""CPU oracle for the five state-space operators (TEST INFRASTRUCTURE ONLY).

This file is a checker, not a product path: only the test-suite, the smoke check
and the CPU-baseline leg of the benchmark may import it.  The shipped operators
never call into it and raise when their CUDA library is missing.

Each function restates, on CPU tensors, the arithmetic of the upstream package's
pure-PyTorch operator of the same name (``src/ssm/ops/python/reference.py`` in
b-vitamins/ssm; the line ranges are given per function).  The restatement is
differentiable, so ``torch.autograd`` on it is the gradient oracle.  Parity of
this file with the upstream implementation is pinned by ``tests/test_oracle_pins.py``
against (a) the known-answer vectors the upstream test-suite ships and (b)
fixtures produced by running the upstream Python operators themselves
(``tests/golden/make_fixtures.py``).

``ssd_scan`` has no upstream function of its own name: the upstream "SSD" operator
has no ``d_state`` axis.  Its oracle is the selective-scan recurrence applied per
head with the state laid out ``(B, H, P, N)``; the fixtures pin it both to the
upstream ``selective_scan`` evaluated on the flattened ``H*P`` channels and to
the stored mamba-ssm ``ssd_combined`` vectors.
"""

from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn.functional as F

Tensor = torch.Tensor

_HALF = (torch.float16, torch.bfloat16)


def _work_dtype(t: Tensor, A: Optional[Tensor] = None) -> torch.dtype:
    """fp16/bf16 compute in fp32, everything else in its own precision; a wider
    ``A`` widens the computation (reference.py:9-19, 135-137)."""
    dt = torch.float32 if t.dtype in _HALF else t.dtype
    if A is not None and A.dtype != torch.float32 and A.dtype != dt:
        dt = torch.promote_types(dt, A.dtype)
    return dt


def _scan_coeff(name: str, p: Tensor, nb: int, nd: int, nn: int, nl: int, dt: torch.dtype):
    """Return ``f(t) -> (B, D, N)`` for the three accepted layouts of the scan's
    input/output projections (reference.py:22-56)."""
    if p.dim() == 2:
        if tuple(p.shape) != (nd, nn):
            raise ValueError(f"{name} must have shape (D, N).")
        const = p.to(dt).unsqueeze(0)
        return lambda t: const
    if p.dim() == 3:
        if tuple(p.shape) != (nb, nd, nn):
            raise ValueError(f"{name} must have shape (B, D, N) when 3-D.")
        const = p.to(dt)
        return lambda t: const
    if p.dim() == 4:
        if p.shape[0] != nb or p.shape[-1] != nl:
            raise ValueError(f"{name} must have shape (B, G, N, L) when 4-D.")
        g = p.shape[1]
        if nd % g != 0:
            raise ValueError("Group dimension must divide D.")
        if p.shape[2] != nn:
            raise ValueError(f"{name} has mismatched state dimension.")
        rep = nd // g
        pw = p.to(dt)
        return lambda t: pw[:, :, :, t].repeat_interleave(rep, dim=1)
    raise ValueError(f"Unsupported rank for {name}.")


def selective_scan(
    u: Tensor,
    delta: Tensor,
    A: Tensor,
    B: Tensor,
    C: Tensor,
    D: Optional[Tensor] = None,
    z: Optional[Tensor] = None,
    dt_bias: Optional[Tensor] = None,
    softplus: bool = False,
    return_last_state: bool = False,
    initial_state: Optional[Tensor] = None,
    keep_state_dtype: bool = False,
):
    """Mamba-1 selective scan, token by token (reference.py:87-194).

    ``h_t = exp(dt_t A) * h_{t-1} + dt_t * B_t * u_t``; ``y_t = <C_t, h_t> + D u_t``;
    ``y_t *= silu(z_t)``.  ``initial_state`` (B, D, N) and ``keep_state_dtype`` (return
    the final state in the compute dtype instead of ``u.dtype``) are additive
    extensions with no upstream counterpart; the defaults reproduce upstream.
    """
    if u.ndim != 3 or delta.ndim != 3:
        raise ValueError("u and delta must have shape (B, D, L).")
    nb, nd, nl = u.shape
    if tuple(delta.shape) != (nb, nd, nl):
        raise ValueError("delta must match the shape of u.")
    nn = A.shape[-1]
    if tuple(A.shape) != (nd, nn):
        raise ValueError("A must have shape (D, N).")
    wd = _work_dtype(u, A)
    uw, dw, Aw = u.to(wd), delta.to(wd), A.to(wd)
    Bt = _scan_coeff("B", B, nb, nd, nn, nl, wd)
    Ct = _scan_coeff("C", C, nb, nd, nn, nl, wd)
    if D is not None and tuple(D.shape) != (nd,):
        raise ValueError("D must have shape (D,).")
    if z is not None and tuple(z.shape) != (nb, nd, nl):
        raise ValueError("z must have shape (B, D, L).")
    if dt_bias is not None:
        if tuple(dt_bias.shape) != (nd,):
            raise ValueError("dt_bias must have shape (D,).")
        dw = dw + dt_bias.to(wd)[None, :, None]
    if softplus:
        dw = F.softplus(dw)
    if initial_state is None:
        h = torch.zeros(nb, nd, nn, dtype=wd)
    else:
        if tuple(initial_state.shape) != (nb, nd, nn):
            raise ValueError("initial_state must have shape (B, D, N).")
        h = initial_state.to(wd)
    cols = []
    for t in range(nl):
        d_t = dw[:, :, t]
        h = torch.exp(d_t[:, :, None] * Aw[None]) * h + (d_t * uw[:, :, t])[:, :, None] * Bt(t)
        cols.append((h * Ct(t)).sum(-1))
    y = torch.stack(cols, dim=-1) if cols else torch.zeros(nb, nd, 0, dtype=wd)
    if D is not None:
        y = y + D.to(wd)[None, :, None] * uw
    if z is not None:
        y = y * F.silu(z.to(wd))
    y = y.to(u.dtype)
    if return_last_state:
        return y, (h if keep_state_dtype else h.to(u.dtype))
    return y


def selective_state_step(
    state: Tensor,
    x: Tensor,
    dt: Tensor,
    A: Tensor,
    B: Tensor,
    C: Tensor,
    D: Optional[Tensor] = None,
    z: Optional[Tensor] = None,
    dt_bias: Optional[Tensor] = None,
    softplus: bool = True,
    inplace: bool = True,
):
    """One decode token of the selective scan with an explicit state that is
    overwritten in place (reference.py:197-309).  With ``inplace=False`` the new
    state is returned as a second value instead (used for gradient checks)."""
    if state.ndim != 3:
        raise ValueError("state must have shape (B, D, N).")
    if x.ndim != 2 or dt.ndim != 2:
        raise ValueError("x and dt must have shape (B, D).")
    nb, nd, nn = state.shape
    if tuple(x.shape) != (nb, nd) or tuple(dt.shape) != (nb, nd):
        raise ValueError("x and dt must match the first two dimensions of state.")
    if tuple(A.shape) != (nd, nn):
        raise ValueError("A must have shape (D, N).")
    wd = _work_dtype(state, A)

    def coeff(name: str, p: Tensor) -> Tensor:
        if p.dim() == 2:
            if tuple(p.shape) != (nd, nn):
                raise ValueError(f"{name} must have shape (D, N).")
            return p.to(wd)[None]
        if p.dim() == 3 and p.shape[0] == nb:
            if p.shape[2] != nn:
                raise ValueError(f"{name} must have matching state dimension.")
            if p.shape[1] == nd:
                return p.to(wd)
            if nd % p.shape[1] != 0:
                raise ValueError(f"{name} group dimension must divide D.")
            return p.to(wd).repeat_interleave(nd // p.shape[1], dim=1)
        raise ValueError(f"{name} must have shape (D, N), (B, D, N) or (B, G, N).")

    Bw, Cw = coeff("B", B), coeff("C", C)
    if D is not None and tuple(D.shape) != (nd,):
        raise ValueError("D must have shape (D,).")
    if z is not None and tuple(z.shape) != (nb, nd):
        raise ValueError("z must have shape (B, D).")
    dtw = dt.to(wd)
    if dt_bias is not None:
        if tuple(dt_bias.shape) != (nd,):
            raise ValueError("dt_bias must have shape (D,).")
        dtw = dtw + dt_bias.to(wd)[None]
    if softplus:
        dtw = F.softplus(dtw)
    xw = x.to(wd)
    new = torch.exp(dtw[:, :, None] * A.to(wd)[None]) * state.to(wd) + (dtw * xw)[:, :, None] * Bw
    y = (new * Cw).sum(-1)
    if D is not None:
        y = y + D.to(wd)[None] * xw
    if z is not None:
        y = y * F.silu(z.to(wd))
    if inplace:
        with torch.no_grad():
            state.copy_(new.to(state.dtype))
        return y.to(x.dtype)
    return y.to(x.dtype), new.to(state.dtype)


def _lengths_from_meta(seq_meta: Optional[dict[str, Any]], nb: int, nl: int) -> list[int]:
    """Valid length per batch row (reference.py:413-428)."""
    if seq_meta is None:
        return [nl] * nb
    if seq_meta.get("cu_seqlens") is not None:
        cu = torch.as_tensor(seq_meta["cu_seqlens"]).to(torch.long)
        if cu.numel() != nb + 1:
            raise ValueError("cu_seqlens must have length B + 1.")
        return [int(v) for v in (cu[1:] - cu[:-1])]
    if seq_meta.get("seq_lens") is not None:
        sl = torch.as_tensor(seq_meta["seq_lens"]).to(torch.long)
        if sl.numel() != nb:
            raise ValueError("seq_lens must have length B.")
        return [int(v) for v in sl]
    raise ValueError("seq_meta must provide cu_seqlens or seq_lens.")


def ssd_chunk_scan(
    X: Tensor,
    dt: Tensor,
    A: Tensor,
    B: Tensor,
    C: Tensor,
    chunk_size: int,
    D: Optional[Tensor] = None,
    z: Optional[Tensor] = None,
    seq_meta: Optional[dict[str, Any]] = None,
    initial_states: Optional[Tensor] = None,
) -> Tensor:
    """Element-wise diagonal recurrence over ``(B, L, H, P)`` (reference.py:312-463):
    ``s_t = exp(dt_t A) s_{t-1} + dt_t B_t X_t``; ``y_t = s_t C_t + D X_t``;
    ``y_t *= silu(z_t)``; rows beyond a sequence's valid length are zero.  The chunk
    size has no numerical effect upstream, and none here."""
    if X.ndim != 4:
        raise ValueError("X must have shape (B, L, H, P).")
    if dt.ndim != 3:
        raise ValueError("dt must have shape (B, L, H).")
    nb, nl, nh, npj = X.shape
    if tuple(dt.shape) != (nb, nl, nh):
        raise ValueError("dt must align with (B, L, H).")
    if int(chunk_size) <= 0:
        raise ValueError("chunk_size must be positive.")
    wd = _work_dtype(X, A)
    if A.ndim == 1:
        if A.shape[0] != nh:
            raise ValueError("A must have shape (H,) when 1-D.")
        Aw = A.to(wd)[:, None].expand(nh, npj)
    elif A.ndim == 2:
        if tuple(A.shape) != (nh, npj):
            raise ValueError("A must have shape (H, P) when 2-D.")
        Aw = A.to(wd)
    else:
        raise ValueError("A must be 1-D or 2-D.")

    def coeff(name: str, p: Tensor):
        if p.dim() == 2:
            if tuple(p.shape) != (nh, npj):
                raise ValueError(f"{name} must have shape (H, P).")
            c = p.to(wd)[None]
            return lambda t: c
        if p.dim() == 3:
            if tuple(p.shape) != (nb, nh, npj):
                raise ValueError(f"{name} must be (B, H, P) when 3-D.")
            c = p.to(wd)
            return lambda t: c
        if p.dim() == 4:
            if tuple(p.shape) != (nb, nl, nh, npj):
                raise ValueError(f"{name} must have shape (B, L, H, P) when 4-D.")
            c = p.to(wd)
            return lambda t: c[:, t]
        raise ValueError(f"Unsupported rank for {name}.")

    Bt, Ct = coeff("B", B), coeff("C", C)
    Dw = None
    if D is not None:
        if D.ndim == 1 and D.shape[0] == nh:
            Dw = D.to(wd)[None, :, None]
        elif D.ndim == 2 and tuple(D.shape) == (nh, npj):
            Dw = D.to(wd)[None]
        else:
            raise ValueError("D must have shape (H,) or (H, P).")
    zw = None
    if z is not None:
        if z.ndim == 3 and tuple(z.shape) == (nb, nl, nh):
            zw = z.to(wd)[..., None]
        elif z.ndim == 4 and tuple(z.shape) == (nb, nl, nh, npj):
            zw = z.to(wd)
        else:
            raise ValueError("z must have shape (B, L, H) or (B, L, H, P).")
    if initial_states is not None:
        if tuple(initial_states.shape) != (nb, nh, npj):
            raise ValueError("initial_states must have shape (B, H, P).")
        s = initial_states.to(wd)
    else:
        s = torch.zeros(nb, nh, npj, dtype=wd)
    lens = torch.tensor(_lengths_from_meta(seq_meta, nb, nl), dtype=torch.long)
    Xw, dtw = X.to(wd), dt.to(wd)
    rows = []
    for t in range(nl):
        d_t = dtw[:, t][..., None]
        s = torch.exp(d_t * Aw[None]) * s + d_t * Bt(t) * Xw[:, t]
        y = s * Ct(t)
        if Dw is not None:
            y = y + Dw * Xw[:, t]
        if zw is not None:
            y = y * F.silu(zw[:, t])
        live = (t < lens).to(wd)[:, None, None]
        rows.append(y * live)
    Y = torch.stack(rows, dim=1) if rows else torch.zeros(nb, 0, nh, npj, dtype=wd)
    return Y.to(X.dtype)


def dw_causal_conv(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, activation: str = "silu") -> Tensor:
    """Depthwise causal 1-D convolution with left padding ``K-1`` and optional SiLU;
    the layout ``(B, C, L)`` or ``(B, L, C)`` is chosen by which axis matches the
    weight's channel count, channels-first winning ties (reference.py:466-537)."""
    if x.ndim != 3:
        raise ValueError("x must have shape (B, C, L) or (B, L, C).")
    nc = weight.shape[0]
    if x.shape[1] == nc:
        first = True
    elif x.shape[2] == nc:
        first = False
    else:
        raise ValueError("weight channel dimension must match x.")
    if weight.ndim == 3:
        if weight.shape[1] != 1:
            raise ValueError("Expected depthwise weights with shape (C, 1, K).")
        w2 = weight[:, 0, :]
    elif weight.ndim == 2:
        w2 = weight
    else:
        raise ValueError("weight must have 2 or 3 dimensions.")
    if bias is not None and tuple(bias.shape) != (nc,):
        raise ValueError("bias must have shape (C,).")
    act = activation.lower()
    if act not in ("silu", "swish", "identity", "none"):
        raise ValueError(f"Unsupported activation '{activation}'.")
    wd = _work_dtype(x)
    xc = (x if first else x.transpose(1, 2)).to(wd)
    nl, k = xc.shape[-1], w2.shape[1]
    xp = F.pad(xc, (k - 1, 0))
    ww = w2.to(wd)
    acc = torch.zeros_like(xc)
    for j in range(k):  # tap j multiplies x[t - (K-1) + j]
        acc = acc + ww[None, :, j, None] * xp[:, :, j : j + nl]
    if bias is not None:
        acc = acc + bias.to(wd)[None, :, None]
    if act in ("silu", "swish"):
        acc = F.silu(acc)
    out = acc.to(x.dtype)
    return out if first else out.transpose(1, 2)


def dw_causal_conv_update(conv_state: Tensor, x: Tensor, weight: Tensor, bias: Optional[Tensor] = None,
                          activation: str = "silu") -> Tensor:
    """Decode-time conv of upstream's ``Mamba1.step`` (modules/mamba1.py:345-353): roll the ``(B, C, K)``
    state left by one in place, append ``x (B, C)``, return ``act(bias + <state, weight>)``."""
    conv_state.copy_(torch.roll(conv_state, shifts=-1, dims=-1))
    conv_state[:, :, -1] = x.to(conv_state.dtype)
    w2 = weight[:, 0, :] if weight.ndim == 3 else weight
    out = (conv_state.float() * w2.float().unsqueeze(0)).sum(dim=-1)
    if bias is not None:
        out = out + bias.float()
    if str(activation).lower() in ("silu", "swish"):
        out = torch.nn.functional.silu(out)
    return out.to(x.dtype)


def fused_layer_norm(
    x: Tensor,
    weight: Tensor,
    bias: Optional[Tensor],
    residual: Optional[Tensor] = None,
    is_rms: bool = False,
    eps: float = 1e-5,
    prenorm: bool = True,
    residual_in_fp32: bool = True,
    return_residual: bool = False,
):
    """Residual add fused with LayerNorm / RMSNorm (reference.py:540-609).
    ``prenorm``: normalise ``x + residual``; otherwise normalise ``x`` and add the
    residual afterwards.  ``return_residual`` (additive extension) also returns the
    summed stream ``x + residual`` in the base dtype."""
    if x.ndim != 3:
        raise ValueError("x must have shape (B, L, D).")
    if tuple(weight.shape) != (x.shape[-1],):
        raise ValueError("weight must match the last dimension of x.")
    if bias is not None and tuple(bias.shape) != (x.shape[-1],):
        raise ValueError("bias must match the last dimension of x.")
    if residual is not None and residual.shape != x.shape:
        raise ValueError("residual must match the shape of x.")
    wd = _work_dtype(x)
    base = torch.float32 if (residual_in_fp32 and residual is not None) else wd
    v = x.to(base)
    r = residual.to(base) if residual is not None else None
    s = v + r if (r is not None and prenorm) else v
    if is_rms:
        n = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps)
    else:
        c = s - s.mean(-1, keepdim=True)
        n = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps)
    y = n * weight.to(n.dtype)
    if bias is not None:
        y = y + bias.to(n.dtype)
    if r is not None and not prenorm:
        y = y + r.to(y.dtype)
    y = y.to(x.dtype)
    if return_residual:
        return y, (v + r if r is not None else v)
    return y


def ssd_scan(
    X: Tensor,
    dt: Tensor,
    A: Tensor,
    B: Tensor,
    C: Tensor,
    chunk_size: int = 256,
    D: Optional[Tensor] = None,
    z: Optional[Tensor] = None,
    dt_bias: Optional[Tensor] = None,
    dt_softplus: bool = False,
    initial_states: Optional[Tensor] = None,
    return_final_states: bool = False,
    cu_seqlens: Optional[Tensor] = None,
    seq_reset: bool = True,
    return_varlen_states: bool = False,
):
    """State-space-dual scan with a ``d_state`` axis (Mamba-2 layout).

    ``cu_seqlens (S + 1,)`` marks ``S`` sequences packed along ``L`` of a batch of one.  The
    ``varlen_states (S, H, P, N)`` are the states after the last token of every sequence, each
    scanned from zero.  With ``seq_reset`` the state behind ``Y`` restarts at every boundary too;
    without it ``Y`` runs through the boundaries, which is what upstream mamba-ssm computes when
    it is given ``cu_seqlens`` but no ``seq_idx`` (its ``combined_varlen`` vector).

    ``X (B,L,H,P)``, ``dt (B,L,H)``, ``A (H,)``, ``B/C (B,L,G,N)`` with ``G | H``,
    ``D (H,)`` or ``(H,P)``, ``z (B,L,H,P)``, state ``(B,H,P,N)`` in fp32.  It is the
    recurrence of reference.py:173-188 applied to channel ``h*P+p`` with
    ``delta[b,h*P+p,t] = dt[b,t,h]`` and ``A[h*P+p,:] = A[h]``; the chunk size does
    not change the result.
    """
    if X.ndim != 4 or dt.ndim != 3:
        raise ValueError("X must be (B, L, H, P) and dt (B, L, H).")
    nb, nl, nh, npj = X.shape
    if tuple(dt.shape) != (nb, nl, nh):
        raise ValueError("dt must align with (B, L, H).")
    if tuple(A.shape) != (nh,):
        raise ValueError("A must have shape (H,).")
    if B.ndim != 4 or B.shape[0] != nb or B.shape[1] != nl or B.shape != C.shape:
        raise ValueError("B and C must have shape (B, L, G, N).")
    ng, nn = B.shape[2], B.shape[3]
    if nh % ng != 0:
        raise ValueError("Group dimension must divide H.")
    wd = _work_dtype(X, A)
    rep = nh // ng
    Xw, dtw, Aw = X.to(wd), dt.to(wd), A.to(wd)
    Bw = B.to(wd).repeat_interleave(rep, dim=2)
    Cw = C.to(wd).repeat_interleave(rep, dim=2)
    if dt_bias is not None:
        dtw = dtw + dt_bias.to(wd)[None, None]
    if dt_softplus:
        dtw = F.softplus(dtw)
    if initial_states is not None:
        if tuple(initial_states.shape) != (nb, nh, npj, nn):
            raise ValueError("initial_states must have shape (B, H, P, N).")
        s = initial_states.to(wd)
    else:
        s = torch.zeros(nb, nh, npj, nn, dtype=wd)
    starts, ends = set(), {}
    if cu_seqlens is not None:
        cu = [int(v) for v in torch.as_tensor(cu_seqlens).tolist()]
        if nb != 1:
            raise ValueError("cu_seqlens needs a batch of one (sequences packed along L).")
        if len(cu) < 2 or cu[0] != 0 or cu[-1] != nl or any(b < a for a, b in zip(cu, cu[1:])):
            raise ValueError("cu_seqlens must rise from 0 to L.")
        starts = set(cu[1:-1])
        ends = {e - 1: k for k, e in enumerate(cu[1:]) if e > cu[k]}
    sr = torch.zeros_like(s)  # the per-sequence state: always restarts at a boundary
    varlen = [torch.zeros(nh, npj, nn, dtype=wd) for _ in range(len(ends) and len(cu) - 1)]
    rows = []
    for t in range(nl):
        d_t = dtw[:, t]
        if t in starts:
            sr = torch.zeros_like(sr)
            if seq_reset:
                s = torch.zeros_like(s)
        decay = torch.exp(d_t * Aw[None])[:, :, None, None]
        inp = (d_t[:, :, None] * Xw[:, t])[..., None] * Bw[:, t][:, :, None, :]
        s = decay * s + inp
        if cu_seqlens is not None:
            sr = decay * sr + inp
            if t in ends:
                varlen[ends[t]] = sr[0]
        rows.append((s * Cw[:, t][:, :, None, :]).sum(-1))
    Y = torch.stack(rows, dim=1) if rows else torch.zeros(nb, 0, nh, npj, dtype=wd)
    if D is not None:
        Dw = D.to(wd)
        Y = Y + (Dw[None, None, :, None] if D.ndim == 1 else Dw[None, None]) * Xw
    if z is not None:
        Y = Y * F.silu(z.to(wd))
    Y = Y.to(X.dtype)
    out = [Y]
    if return_final_states:
        out.append(s.to(torch.float32) if wd != torch.float64 else s)
    if return_varlen_states:
        if cu_seqlens is None:
            raise ValueError("return_varlen_states needs cu_seqlens.")
        v = torch.stack(varlen) if varlen else torch.zeros(0, nh, npj, nn, dtype=wd)
        out.append(v.to(torch.float32) if wd != torch.float64 else v)
    return out[0] if len(out) == 1 else tuple(out)


def softplus_threshold() -> float:
    """``torch.nn.functional.softplus`` switches to the identity above this input."""
    return 20.0


def silu(v: float) -> float:
    return v / (1.0 + math.exp(-v))
