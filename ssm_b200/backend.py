"""Drop-in object for the upstream package's compiled-CUDA-backend slot.

Upstream's façade (src/ssm/ops/__init__.py:85-109) caches its CUDA extension module in the
global ``ssm.ops._CUDA_OPS`` and calls ten functions on it whose names, argument order,
defaults and return tuples are fixed by src/ssm/ops/cuda/bindings.cpp:96-152.  ``Backend``
provides exactly those ten callables on top of the C-ABI library, and ``install()`` stores an
instance in that slot, so that ``ssm.ops.selective_scan`` etc. dispatch CUDA tensors to the
sm_100a kernels with no change to upstream code.  Errors raised as ``ValueError`` here pass
through upstream's ``RuntimeError -> ValueError`` translation unchanged.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops as O

Tensor = torch.Tensor


class Backend:
    """The ten entry points of upstream's ``ssm_cuda_ops`` extension module."""

    # -- selective scan ---------------------------------------------------------------
    def selective_scan(self, u, delta, A, B, C, D=None, z=None, dt_bias=None, softplus=False, return_last_state=False):
        """-> (out, last_state, cache); ``last_state`` is empty unless requested, ``cache``
        holds the state checkpoints the backward call consumes."""
        sc = O._ScanCtx(u, delta, A, B, C, D, z, dt_bias, softplus, None)
        out, last, ck = O._scan_forward(sc, bool(return_last_state), True, u.dtype)
        if last is None:
            last = torch.empty(0, dtype=u.dtype, device=u.device)
        return out, last, ck

    def selective_scan_backward(self, grad_output, grad_last_state, u, delta, A, B, C, D=None, z=None, dt_bias=None,
                                softplus=False, forward_output=None, cache=None):
        """-> (du, ddelta, dA, dB, dC, dD?, dz?, ddt_bias?) in the dtypes / shapes of the inputs."""
        sc = O._ScanCtx(u, delta, A, B, C, D, z, dt_bias, softplus, None)
        if cache is None or cache.numel() == 0:
            _, _, cache = O._scan_forward(sc, False, True, u.dtype)
        du, dd, dA, dB, dC, dD, dz, db = O._scan_backward(sc, cache, grad_output, grad_last_state, B, C)
        return (
            du, dd.to(delta.dtype), dA.to(A.dtype), dB, dC,
            None if D is None else dD.to(D.dtype),
            None if z is None else dz.to(z.dtype),
            None if dt_bias is None else db.to(dt_bias.dtype),
        )

    # -- state step ---------------------------------------------------------------------
    def selective_state_step(self, state, x, dt, A, B, C, D=None, z=None, dt_bias=None, softplus=True):
        sc = O._StepCtx(state, x, dt, A, B, C, D, z, dt_bias, softplus)
        return O._step_forward(sc, state)

    def selective_state_step_backward(self, grad_output, grad_state, state, x, dt, A, B, C, D=None, z=None, dt_bias=None,
                                      softplus=True):
        """-> (dstate, dx, ddt, dA, dB, dC, dD?, dz?, ddt_bias?); ``state`` is the state before the step."""
        leaves = [t.detach().clone().requires_grad_(True) if t is not None else None for t in (state, x, dt, A, B, C, D, z, dt_bias)]
        with torch.enable_grad():
            y, new = O._StateStepFn.apply(*leaves, softplus)
        gs = torch.zeros_like(new) if grad_state is None else grad_state
        live = [t for t in leaves if t is not None]
        grads = iter(torch.autograd.grad((y, new), live, (grad_output, gs), allow_unused=True))
        return tuple(None if t is None else next(grads) for t in leaves)

    # -- element-wise chunk scan ----------------------------------------------------------
    def ssd_chunk_scan(self, X, dt, A, B, C, chunk_size, D=None, z=None, seq_lens=None, cu_seqlens=None, initial_states=None):
        meta = _meta(seq_lens, cu_seqlens)
        cc = O._ChunkCtx(X, dt, A, B, C, chunk_size, D, z, meta, initial_states)
        return O._chunk_forward(cc)[0]

    def ssd_chunk_scan_backward(self, grad_output, X, dt, A, B, C, chunk_size, D=None, z=None, seq_lens=None, cu_seqlens=None,
                                initial_states=None):
        """-> (dX, ddt, dA, dB, dC, dD?, dz?, dinitial?)."""
        meta = _meta(seq_lens, cu_seqlens)
        leaves = [t.detach().clone().requires_grad_(True) if t is not None else None for t in (X, dt, A, B, C, D, z, initial_states)]
        with torch.enable_grad():
            Y = O._ChunkScanFn.apply(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], chunk_size, leaves[5], leaves[6], meta, leaves[7])
        live = [t for t in leaves if t is not None]
        grads = iter(torch.autograd.grad(Y, live, grad_output, allow_unused=True))
        return tuple(None if t is None else next(grads) for t in leaves)

    # -- depthwise causal conv -----------------------------------------------------------
    def dw_causal_conv(self, x, weight, bias=None, activation="silu"):
        with torch.no_grad():
            return O.dw_causal_conv(x, weight, bias, activation)

    def dw_causal_conv_backward(self, grad_output, x, weight, bias=None, activation="silu"):
        """-> (dx, dw, db?)."""
        leaves = [t.detach().clone().requires_grad_(True) if t is not None else None for t in (x, weight, bias)]
        with torch.enable_grad():
            y = O.dw_causal_conv(leaves[0], leaves[1], leaves[2], activation)
        live = [t for t in leaves if t is not None]
        grads = iter(torch.autograd.grad(y, live, grad_output, allow_unused=True))
        return tuple(None if t is None else next(grads) for t in leaves)

    # -- fused add + norm ----------------------------------------------------------------
    def fused_layer_norm(self, x, weight, bias=None, residual=None, is_rms=False, eps=1e-5, prenorm=True, residual_in_fp32=True):
        with torch.no_grad():
            return O.fused_layer_norm(x, weight, bias, residual, is_rms, eps, prenorm, residual_in_fp32)

    def fused_layer_norm_backward(self, grad_output, x, weight, bias=None, residual=None, is_rms=False, eps=1e-5, prenorm=True,
                                  residual_in_fp32=True):
        """-> (dx, dw, db, dres); absent inputs give empty tensors, as upstream's extension does."""
        leaves = [t.detach().clone().requires_grad_(True) if t is not None else None for t in (x, weight, bias, residual)]
        with torch.enable_grad():
            y = O.fused_layer_norm(leaves[0], leaves[1], leaves[2], leaves[3], is_rms, eps, prenorm, residual_in_fp32)
        live = [t for t in leaves if t is not None]
        grads = iter(torch.autograd.grad(y, live, grad_output, allow_unused=True))
        out = [None if t is None else next(grads) for t in leaves]
        empty = torch.empty(0, dtype=x.dtype, device=x.device)
        return tuple(empty if g is None else g for g in out)


def _meta(seq_lens: Optional[Tensor], cu_seqlens: Optional[Tensor]):
    if cu_seqlens is not None:
        return {"cu_seqlens": cu_seqlens}
    if seq_lens is not None:
        return {"seq_lens": seq_lens}
    return None


def install(ssm_ops_module=None) -> Backend:
    """Put a :class:`Backend` into upstream's ``ssm.ops._CUDA_OPS`` slot (and clear a cached
    load failure).  Pass the module explicitly or let it be imported as ``ssm.ops``."""
    from . import _lib

    _lib.load()  # fail now, loudly, if the CUDA library is not built
    if ssm_ops_module is None:
        import importlib

        ssm_ops_module = importlib.import_module("ssm.ops")
    be = Backend()
    ssm_ops_module._CUDA_OPS = be
    ssm_ops_module._CUDA_LOAD_ERROR = None
    return be
