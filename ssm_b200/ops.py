"""The five state-space operators on the B200 CUDA library, with the upstream signatures.

``selective_scan``, ``selective_state_step``, ``ssd_chunk_scan``, ``dw_causal_conv`` and
``fused_layer_norm`` take the arguments of ``ssm.ops`` in b-vitamins/ssm
(src/ssm/ops/__init__.py:1255-1690; semantics src/ssm/ops/python/reference.py), accept CUDA
tensors only, and are differentiable through ``torch.autograd.Function`` wrappers whose
forward and backward both run hand-written sm_100a kernels behind the C ABI of
``include/ssm_b200.h``.  Contract violations raise ``ValueError`` as upstream does.  There is
no CPU path and no PyTorch fallback: a missing library or a CPU tensor is an error.

Additive keyword arguments that upstream does not have are marked "extension" below; their
defaults reproduce upstream behaviour.
"""

from __future__ import annotations

import ctypes as C
import math
from typing import Any, Optional

import torch
import torch.nn.functional as F

from . import _lib as L

Tensor = torch.Tensor

_CODES = {torch.float32: L.F32, torch.bfloat16: L.BF16, torch.float16: L.F16}


def _code(t: Tensor, what: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise ValueError(f"{what}: dtype {t.dtype} is not built (float32, bfloat16 and float16 are)") from None


def _need_cuda(*ts: Optional[Tensor]) -> torch.device:
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("ssm_b200 operators run on CUDA tensors only; there is no CPU fallback")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("all tensors must be on the same CUDA device")
    assert dev is not None
    return dev


def _p(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _f32(t: Optional[Tensor]) -> Optional[Tensor]:
    if t is None:
        return None
    return t.detach().to(torch.float32).contiguous()


def _c(t: Optional[Tensor]) -> Optional[Tensor]:
    if t is None:
        return None
    t = t.detach()
    return t if t.is_contiguous() else t.contiguous()


def _rows(t: Tensor) -> Tensor:
    """A (B, D, L) activation in one of the two row layouts the kernels address directly: dense
    (B, D, L), or a dense (D, B, L) buffer viewed as (B, D, L).  Anything else is copied to dense."""
    t = t.detach()
    if t.is_contiguous() or (t.dim() == 3 and t.stride(2) == 1 and t.permute(1, 0, 2).is_contiguous()):
        return t
    return t.contiguous()


def _rows_like(t: Optional[Tensor], ref: Tensor) -> Optional[Tensor]:
    """``t`` with the dtype and exactly the strides of ``ref`` (copied only when it differs)."""
    if t is None:
        return None
    t = t.detach()
    if t.dtype == ref.dtype and t.stride() == ref.stride():
        return t
    out = torch.empty_like(ref)
    out.copy_(t)
    return out


def _guard(ctx, *tensors: Optional[Tensor]) -> None:
    """Remember the version counters of the tensors a backward pass will read again; `_check_guard`
    raises if one of them was modified in place in between (what autograd does for saved tensors)."""
    ctx._guarded = [(t, t._version) for t in tensors if t is not None]


def _check_guard(ctx) -> None:
    for t, v in getattr(ctx, "_guarded", ()):
        if t._version != v:
            raise RuntimeError("one of the tensors needed for the backward pass of an ssm_b200 operator has been modified in place "
                               f"(shape {tuple(t.shape)}, version {t._version}, expected {v})")


class _DeviceStatus:
    """The device word that the tensor-core kernels set when one of their bounded waits runs out, with a pinned host
    mirror.  After every launch the word is copied to the mirror asynchronously on the launching stream; `poll` reads
    the mirror once that copy has finished, so a timed-out wait surfaces at the next call without the hot path ever
    synchronising.  `poll(sync=True)` waits for the last launch first."""

    _per_device: dict[int, "_DeviceStatus"] = {}

    def __init__(self, device: torch.device):
        self.word = torch.zeros(1, dtype=torch.int32, device=device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event: Optional[torch.cuda.Event] = None

    @classmethod
    def of(cls, device: torch.device) -> "_DeviceStatus":
        idx = device.index if device.index is not None else torch.cuda.current_device()
        st = cls._per_device.get(idx)
        if st is None:
            st = cls._per_device[idx] = cls(torch.device("cuda", idx))
        return st

    def after_launch(self) -> None:
        if torch.cuda.is_current_stream_capturing():
            return
        self.host.copy_(self.word, non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record()

    def poll(self, sync: bool = False) -> None:
        if self.event is None or torch.cuda.is_current_stream_capturing():
            return
        if sync:
            self.event.synchronize()
        elif not self.event.query():
            return
        code = int(self.host[0])
        if code:
            self.host.zero_()
            self.word.zero_()
            self.event = None
            raise RuntimeError(f"ssd_scan: a bounded device-side wait ran out in an earlier launch (status {code}); its outputs are invalid")


def ssd_check_status(device: Optional[torch.device] = None) -> None:
    """Wait for the last tensor-core SSD launch on ``device`` and raise if one of its bounded waits ran out."""
    _DeviceStatus.of(torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)).poll(sync=True)


def ssd_wait_selftest(probes: int = 100, device: Optional[torch.device] = None) -> None:
    """Launch the library's wait self-test on ``device``: a warp waits on a barrier nothing arms and gives up after ``probes``
    probes, recording status 3 like a tensor-core kernel whose copy never landed.  The next ``ssd_scan`` call (or
    :func:`ssd_check_status`) then raises; the device and the context stay usable."""
    st = _DeviceStatus.of(torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device))
    with torch.cuda.device(st.word.device):
        L.check(L.load().ssm_ssd_wait_selftest(st.word.data_ptr(), int(probes), _stream()))
        st.after_launch()


def _call(fn, args) -> None:
    try:
        L.check(fn(C.byref(args), _stream()))
    except L.BackendError as exc:
        if exc.code < 0:
            raise ValueError(str(exc)) from None
        raise


# =========================================================================================
# selective_scan
# =========================================================================================


def _scan_coeff(name: str, p: Tensor, nb: int, nd: int, nn: int, nl: int):
    """Return (tensor, groups, (sb, sg, sn, st)) for the B / C layouts of reference.py:22-56."""
    if p.dim() == 2:
        if tuple(p.shape) != (nd, nn):
            raise ValueError(f"{name} must have shape (D, N).")
        return _f32(p), nd, (0, nn, 1, 0)
    if p.dim() == 3:
        if tuple(p.shape) != (nb, nd, nn):
            raise ValueError(f"{name} must have shape (B, D, N) when 3-D.")
        return _f32(p), nd, (nd * nn, nn, 1, 0)
    if p.dim() == 4:
        if p.shape[0] != nb or p.shape[-1] != nl:
            raise ValueError(f"{name} must have shape (B, G, N, L) when 4-D.")
        g = p.shape[1]
        if g == 0 or nd % g != 0:
            raise ValueError("Group dimension must divide D.")
        if p.shape[2] != nn:
            raise ValueError(f"{name} has mismatched state dimension.")
        return _c(p), g, (g * nn * nl, nn * nl, nl, 1)
    raise ValueError(f"Unsupported rank for {name}.")


class _ScanCtx:
    """Validated, contiguous inputs of one selective-scan call."""

    def __init__(self, u, delta, A, B, C_, D, z, dt_bias, softplus, initial_state):
        if u.ndim != 3 or delta.ndim != 3:
            raise ValueError("u and delta must have shape (B, D, L).")
        nb, nd, nl = u.shape
        if tuple(delta.shape) != (nb, nd, nl):
            raise ValueError("delta must match the shape of u.")
        if A.ndim != 2 or tuple(A.shape) != (nd, A.shape[-1]):
            raise ValueError("A must have shape (D, N).")
        nn = A.shape[-1]
        if nn < 1 or nn > 256:
            raise ValueError("selective_scan: the state dimension must be in [1, 256].")
        if A.is_complex():
            raise ValueError("selective_scan: complex A is not built")
        _need_cuda(u, delta, A, B, C_, D, z, dt_bias, initial_state)
        self.io = _code(u, "selective_scan")
        self.shape = (nb, nd, nl, nn)
        self.u = _rows(u)
        self.delta = _rows_like(delta, self.u)
        self.A = _f32(A)
        Bt, gb, sB = _scan_coeff("B", B, nb, nd, nn, nl)
        Ct, gc, sC = _scan_coeff("C", C_, nb, nd, nn, nl)
        if gb != gc:
            # differing group counts: expand the coarser one so that one group map serves both
            g = max(gb, gc)
            if g % min(gb, gc) != 0:
                raise ValueError("B and C group dimensions must nest.")
            if gb < g:
                Bt, sB = _regroup(Bt, sB, gb, g, nb, nn, nl)
            else:
                Ct, sC = _regroup(Ct, sC, gc, g, nb, nn, nl)
            gb = g
        if Bt.dtype != Ct.dtype:
            Bt, Ct = Bt.float(), Ct.float()
        _code(Bt, "selective_scan B/C")
        self.B, self.C, self.groups, self.sB, self.sC = Bt, Ct, gb, sB, sC
        if D is not None and tuple(D.shape) != (nd,):
            raise ValueError("D must have shape (D,).")
        if z is not None and tuple(z.shape) != (nb, nd, nl):
            raise ValueError("z must have shape (B, D, L).")
        if dt_bias is not None and tuple(dt_bias.shape) != (nd,):
            raise ValueError("dt_bias must have shape (D,).")
        if initial_state is not None and tuple(initial_state.shape) != (nb, nd, nn):
            raise ValueError("initial_state must have shape (B, D, N).")
        self.D = _f32(D)
        self.z = _rows_like(z, self.u)
        self.dt_bias = _f32(dt_bias)
        self.init = _f32(initial_state)
        self.softplus = bool(softplus)

    def fill(self, a: L.ScanFwdArgs) -> None:
        nb, nd, nl, nn = self.shape
        a.batch, a.dim, a.len, a.nstate = nb, nd, nl, nn
        a.io_dtype, a.bc_dtype = self.io, _CODES[self.B.dtype]
        a.delta_softplus = int(self.softplus)
        a.u, a.delta, a.z, a.A = _p(self.u), _p(self.delta), _p(self.z), _p(self.A)
        a.Bm, a.Cm, a.bc_groups = _p(self.B), _p(self.C), self.groups
        a.b_sb, a.b_sg, a.b_sn, a.b_st = self.sB
        a.c_sb, a.c_sg, a.c_sn, a.c_st = self.sC
        a.D, a.dt_bias, a.initial_state = _p(self.D), _p(self.dt_bias), _p(self.init)
        a.row_sb, a.row_sd = (self.u.stride(0), self.u.stride(1)) if self.u.numel() else (nd * nl, nl)


def _regroup(t: Tensor, strides, g_old: int, g_new: int, nb: int, nn: int, nl: int):
    """Repeat a coarser-grouped (B, G, N, L) coefficient so that it has ``g_new`` groups."""
    if strides[3] == 0:  # (D, N) / (B, D, N) are always per channel; cannot be coarser
        raise ValueError("B and C group dimensions must nest.")
    t = t.repeat_interleave(g_new // g_old, dim=1).contiguous()
    return t, (g_new * nn * nl, nn * nl, nl, 1)


def _scan_forward(ctx: _ScanCtx, want_last: bool, want_ckpt: bool, last_dtype: torch.dtype):
    nb, nd, nl, nn = ctx.shape
    lib = L.load()
    out = torch.empty_like(ctx.u)
    last = torch.empty(nb, nd, nn, dtype=last_dtype, device=ctx.u.device) if want_last else None
    ck = None
    if want_ckpt:
        iv = lib.ssm_scan_checkpoint_interval()
        ck = torch.empty(nb, nd, max(1, (nl + iv - 1) // iv), nn, dtype=torch.float32, device=ctx.u.device)
    a = L.ScanFwdArgs()
    ctx.fill(a)
    a.out, a.last_state, a.checkpoints = _p(out), _p(last), _p(ck)
    nseg = int(lib.ssm_scan_split_segments(nb, nd, nl, nn))  # > 1: too few rows to fill the GPU, the sequence is cut into parallel segments
    split = None
    if nseg > 1:
        split = torch.empty(2 * nb * nd * nseg * nn, dtype=torch.float32, device=ctx.u.device)
        a.split_scratch, a.split_segments = _p(split), nseg
    a.last_dtype = _CODES[last_dtype] if want_last else 0
    _call(lib.ssm_selective_scan_fwd, a)
    return out, last, ck


def _scan_backward(ctx: _ScanCtx, ck: Tensor, grad_out: Tensor, grad_last: Optional[Tensor], B_like: Tensor, C_like: Tensor,
                   want_dinit: bool = False):
    nb, nd, nl, nn = ctx.shape
    lib = L.load()
    dev = ctx.u.device
    dinit = None
    if want_dinit:
        # an empty sequence hands the gradient of the last state straight to the initial state
        dinit = torch.zeros(nb, nd, nn, dtype=torch.float32, device=dev) if (nl == 0 and grad_last is None) else \
            (grad_last.detach().float().clone() if nl == 0 else torch.empty(nb, nd, nn, dtype=torch.float32, device=dev))
    du = torch.empty_like(ctx.u)
    ddelta = torch.empty_like(ctx.u)
    dz = torch.empty_like(ctx.u) if ctx.z is not None else None
    dA = torch.zeros(nd, nn, dtype=torch.float32, device=dev)
    # gradient buffers in the layout of the (contiguous) coefficients the kernel read
    dB = torch.zeros(ctx.B.shape, dtype=torch.float32, device=dev)
    dC = torch.zeros(ctx.C.shape, dtype=torch.float32, device=dev)
    dD = torch.zeros(nd, dtype=torch.float32, device=dev) if ctx.D is not None else None
    dbias = torch.zeros(nd, dtype=torch.float32, device=dev) if ctx.dt_bias is not None else None
    g = L.ScanBwdArgs()
    ctx.fill(g.fwd)
    g.fwd.checkpoints = _p(ck)
    go = _rows_like(grad_out, ctx.u)
    gl = _f32(grad_last)
    g.dout, g.dlast_state = _p(go), _p(gl)
    g.du, g.ddelta, g.dz = _p(du), _p(ddelta), _p(dz)
    g.dA, g.dB, g.dC, g.dD, g.ddt_bias = _p(dA), _p(dB), _p(dC), _p(dD), _p(dbias)
    g.db_sb, g.db_sg, g.db_sn, g.db_st = ctx.sB
    g.dc_sb, g.dc_sg, g.dc_sn, g.dc_st = ctx.sC
    g.dinitial_state = _p(dinit)
    _call(lib.ssm_selective_scan_bwd, g)

    def fold(grad: Tensor, like: Tensor) -> Tensor:
        if grad.shape != like.shape:  # the coefficient had been regrouped: sum the repeats back
            rep = grad.shape[1] // like.shape[1]
            grad = grad.view(like.shape[0], like.shape[1], rep, *like.shape[2:]).sum(2)
        return grad.to(like.dtype)

    if want_dinit:
        return du, ddelta, dA, fold(dB, B_like), fold(dC, C_like), dD, dz, dbias, dinit
    return du, ddelta, dA, fold(dB, B_like), fold(dC, C_like), dD, dz, dbias


class _SelectiveScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, B, C_, D, z, dt_bias, softplus, return_last_state, initial_state, keep_state_fp32):
        sc = _ScanCtx(u, delta, A, B, C_, D, z, dt_bias, softplus, initial_state)
        needs = any(t is not None and t.requires_grad for t in (u, delta, A, B, C_, D, z, dt_bias, initial_state))
        last_dtype = torch.float32 if keep_state_fp32 else u.dtype
        out, last, ck = _scan_forward(sc, return_last_state, needs, last_dtype)
        ctx.sc, ctx.ck = sc, ck
        ctx.like = (B, C_, A, D, z, dt_bias, delta, initial_state)
        _guard(ctx, u, delta, A, B, C_, D, z, dt_bias, initial_state)
        if return_last_state:
            return out, last
        return out

    @staticmethod
    def backward(ctx, grad_out, grad_last=None):
        _check_guard(ctx)
        sc: _ScanCtx = ctx.sc
        B, C_, A, D, z, dt_bias, delta, init = ctx.like
        if grad_out is None:
            grad_out = torch.zeros_like(sc.u)
        want_dinit = init is not None and init.requires_grad
        res = _scan_backward(sc, ctx.ck, grad_out, grad_last, B, C_, want_dinit)
        du, ddelta, dA, dB, dC, dD, dz, dbias = res[:8]
        return (
            du,
            ddelta.to(delta.dtype),
            dA.to(A.dtype),
            dB,
            dC,
            None if D is None else dD.to(D.dtype),
            None if z is None else dz.to(z.dtype),
            None if dt_bias is None else dbias.to(dt_bias.dtype),
            None, None, res[8].to(init.dtype) if want_dinit else None, None,
        )


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
    keep_state_fp32: bool = False,
):
    """Mamba-1 selective scan (upstream ``ssm.ops.selective_scan``, reference.py:87-194).

    Extensions: ``initial_state`` ``(B, D, N)`` starts the recurrence from a given state (it
    receives a gradient like any other input); ``keep_state_fp32`` returns the last state in
    fp32 instead of ``u.dtype``.
    """
    if u.dtype == torch.float64:  # double-precision kernels, meant for gradient checks (ops_f64.py)
        from . import ops_f64
        return ops_f64.selective_scan(u, delta, A, B, C, D, z, dt_bias, softplus, return_last_state, initial_state)
    res = _SelectiveScanFn.apply(u, delta, A, B, C, D, z, dt_bias, softplus, return_last_state, initial_state, keep_state_fp32)
    return res


# =========================================================================================
# selective_state_step
# =========================================================================================


def _step_coeff(name: str, p: Tensor, nb: int, nd: int, nn: int):
    if p.dim() == 2:
        if tuple(p.shape) != (nd, nn):
            raise ValueError(f"{name} must have shape (D, N).")
        return nd, (0, nn, 1)
    if p.dim() == 3 and p.shape[0] == nb:
        g = p.shape[1]
        if p.shape[2] != nn:
            raise ValueError(f"{name} must have matching state dimension.")
        if g == 0 or nd % g != 0:
            raise ValueError(f"{name} group dimension must divide D.")
        return g, (g * nn, nn, 1)
    raise ValueError(f"{name} must have shape (D, N), (B, D, N) or (B, G, N).")


class _StepCtx:
    def __init__(self, state, x, dt, A, B, C_, D, z, dt_bias, softplus):
        if state.ndim != 3:
            raise ValueError("state must have shape (B, D, N).")
        if x.ndim != 2 or dt.ndim != 2:
            raise ValueError("x and dt must have shape (B, D).")
        nb, nd, nn = state.shape
        if tuple(x.shape) != (nb, nd) or tuple(dt.shape) != (nb, nd):
            raise ValueError("x and dt must match the first two dimensions of state.")
        if tuple(A.shape) != (nd, nn):
            raise ValueError("A must have shape (D, N).")
        _need_cuda(state, x, dt, A, B, C_, D, z, dt_bias)
        self.shape = (nb, nd, nn)
        self.io = _code(x, "selective_state_step")
        gb, self.sB = _step_coeff("B", B, nb, nd, nn)
        gc, self.sC = _step_coeff("C", C_, nb, nd, nn)
        Bt, Ct = _c(B), _c(C_)
        if gb != gc or Bt.dtype != Ct.dtype or Bt.dtype not in _CODES:
            # bring both to per-channel fp32 (B, D, N) / (D, N) form
            Bt, gb, self.sB = _expand_step(Bt, gb, nb, nd, nn)
            Ct, gc, self.sC = _expand_step(Ct, gc, nb, nd, nn)
        self.B, self.C, self.groups = Bt, Ct, gb
        if D is not None and tuple(D.shape) != (nd,):
            raise ValueError("D must have shape (D,).")
        if z is not None and tuple(z.shape) != (nb, nd):
            raise ValueError("z must have shape (B, D).")
        if dt_bias is not None and tuple(dt_bias.shape) != (nd,):
            raise ValueError("dt_bias must have shape (D,).")
        self.x, self.dt = _c(x), _c(dt.to(x.dtype))
        self.z = None if z is None else _c(z.to(x.dtype))
        self.A, self.D, self.dt_bias = _f32(A), _f32(D), _f32(dt_bias)
        self.softplus = bool(softplus)

    def fill(self, a: L.StepArgs, state32: Tensor) -> None:
        nb, nd, nn = self.shape
        a.batch, a.dim, a.nstate, a.io_dtype = nb, nd, nn, self.io
        a.bc_dtype, a.bc_groups, a.dt_softplus, a.param_heads = _CODES[self.B.dtype], self.groups, int(self.softplus), 0
        a.state, a.x, a.dt, a.z, a.A = _p(state32), _p(self.x), _p(self.dt), _p(self.z), _p(self.A)
        a.Bm, a.Cm = _p(self.B), _p(self.C)
        a.b_sb, a.b_sg, a.b_sn = self.sB
        a.c_sb, a.c_sg, a.c_sn = self.sC
        a.D, a.dt_bias = _p(self.D), _p(self.dt_bias)


def _expand_step(t: Tensor, g: int, nb: int, nd: int, nn: int):
    t = t.float()
    if t.dim() == 3 and g != nd:
        t = t.repeat_interleave(nd // g, dim=1)
    t = t.contiguous()
    return t, nd, ((0, nn, 1) if t.dim() == 2 else (nd * nn, nn, 1))


def _step_forward(sc: _StepCtx, state: Tensor) -> Tensor:
    """Runs the step; ``state`` is updated in place (through an fp32 copy if it is not fp32)."""
    lib = L.load()
    direct = state.dtype == torch.float32 and state.is_contiguous()
    work = state.detach() if direct else state.detach().float().contiguous()
    out = torch.empty_like(sc.x)
    a = L.StepArgs()
    sc.fill(a, work)
    a.out = _p(out)
    _call(lib.ssm_selective_state_step, a)
    if not direct:
        state.detach().copy_(work)
    return out


class _StateStepFn(torch.autograd.Function):
    """Out-of-place form used when gradients are needed: returns (y, new_state)."""

    @staticmethod
    def forward(ctx, state, x, dt, A, B, C_, D, z, dt_bias, softplus):
        sc = _StepCtx(state, x, dt, A, B, C_, D, z, dt_bias, softplus)
        old = state.detach().float().contiguous()
        new = old.clone()
        y = _step_forward(sc, new)
        ctx.sc, ctx.old = sc, old
        ctx.like = (state, dt, A, B, C_, D, z, dt_bias)
        _guard(ctx, x, dt, A, B, C_, D, z, dt_bias)
        return y, new.to(state.dtype)

    @staticmethod
    def backward(ctx, gy, gstate):
        _check_guard(ctx)
        sc: _StepCtx = ctx.sc
        state, dt, A, B, C_, D, z, dt_bias = ctx.like
        nb, nd, nn = sc.shape
        lib = L.load()
        dev = sc.x.device
        g = L.StepBwdArgs()
        sc.fill(g.fwd, ctx.old)
        gy = torch.zeros_like(sc.x) if gy is None else _c(gy.to(sc.x.dtype))
        gs = _f32(gstate)
        dstate = torch.empty(nb, nd, nn, dtype=torch.float32, device=dev)
        dx, ddt = torch.empty_like(sc.x), torch.empty_like(sc.x)
        dz = torch.empty_like(sc.x) if sc.z is not None else None
        dA = torch.zeros(nd, nn, dtype=torch.float32, device=dev)
        dB = torch.zeros(sc.B.shape, dtype=torch.float32, device=dev)
        dC = torch.zeros(sc.C.shape, dtype=torch.float32, device=dev)
        dD = torch.zeros(nd, dtype=torch.float32, device=dev) if sc.D is not None else None
        db = torch.zeros(nd, dtype=torch.float32, device=dev) if sc.dt_bias is not None else None
        g.dout, g.dnew_state, g.dstate = _p(gy), _p(gs), _p(dstate)
        g.dx, g.ddt, g.dz = _p(dx), _p(ddt), _p(dz)
        g.dA, g.dB, g.dC, g.dD, g.ddt_bias = _p(dA), _p(dB), _p(dC), _p(dD), _p(db)
        _call(lib.ssm_selective_state_step_bwd, g)

        def fold(grad: Tensor, like: Tensor) -> Tensor:
            if grad.shape != like.shape:  # grouped (B, G, N) had been expanded to (B, D, N)
                rep = grad.shape[1] // like.shape[1]
                grad = grad.view(like.shape[0], like.shape[1], rep, like.shape[2]).sum(2)
            return grad.to(like.dtype)

        return (
            dstate.to(state.dtype), dx, ddt.to(dt.dtype), dA.to(A.dtype), fold(dB, B), fold(dC, C_),
            None if D is None else dD.to(D.dtype),
            None if z is None else dz.to(z.dtype),
            None if dt_bias is None else db.to(dt_bias.dtype),
            None,
        )


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
) -> Tensor:
    """One decode token; ``state`` ``(B, D, N)`` is overwritten in place (upstream
    ``ssm.ops.selective_state_step``, reference.py:197-309)."""
    if x.dtype == torch.float64:
        from . import ops_f64
        return ops_f64.selective_state_step(state, x, dt, A, B, C, D, z, dt_bias, softplus)
    if any(t is not None and t.requires_grad for t in (state, x, dt, A, B, C, D, z, dt_bias)) and torch.is_grad_enabled():
        y, new = _StateStepFn.apply(state, x, dt, A, B, C, D, z, dt_bias, softplus)
        with torch.no_grad():
            state.copy_(new)
        return y
    sc = _StepCtx(state, x, dt, A, B, C, D, z, dt_bias, softplus)
    return _step_forward(sc, state)


def selective_state_step_heads(
    state: Tensor, x: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor,
    D: Optional[Tensor] = None, z: Optional[Tensor] = None, dt_bias: Optional[Tensor] = None, softplus: bool = True,
) -> Tensor:
    """Extension: Mamba-2 decode step.  ``state (B, H, P, N)`` fp32 in place, ``x, z (B, H, P)``,
    ``dt (B, H)``, ``A, D, dt_bias (H,)``, ``B, C (B, G, N)``; returns ``(B, H, P)``.  Equivalent to
    the upstream step on ``H*P`` flattened channels with per-head parameters broadcast."""
    if state.ndim != 4 or x.ndim != 3:
        raise ValueError("state must be (B, H, P, N) and x (B, H, P).")
    nb, nh, npj, nn = state.shape
    if tuple(x.shape) != (nb, nh, npj) or tuple(dt.shape) != (nb, nh) or tuple(A.shape) != (nh,):
        raise ValueError("x must be (B, H, P), dt (B, H) and A (H,).")
    if B.ndim != 3 or B.shape != C.shape or B.shape[0] != nb or B.shape[2] != nn or nh % B.shape[1] != 0:
        raise ValueError("B and C must have shape (B, G, N) with G dividing H.")
    _need_cuda(state, x, dt, A, B, C, D, z, dt_bias)
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise ValueError("state must be a contiguous float32 tensor.")
    lib = L.load()
    xs, dts = _c(x), _c(dt.to(x.dtype))
    zs = None if z is None else _c(z.to(x.dtype))
    Bt, Ct = _c(B), _c(C)
    if Bt.dtype != Ct.dtype or Bt.dtype not in _CODES:
        Bt, Ct = Bt.float(), Ct.float()
    A32, D32, b32 = _f32(A), _f32(D), _f32(dt_bias)
    out = torch.empty_like(xs)
    g = Bt.shape[1]
    a = L.StepArgs()
    a.batch, a.dim, a.nstate, a.io_dtype = nb, nh * npj, nn, _code(x, "selective_state_step_heads")
    a.bc_dtype, a.bc_groups, a.dt_softplus, a.param_heads = _CODES[Bt.dtype], g, int(softplus), nh
    a.state, a.x, a.dt, a.z, a.A = _p(state), _p(xs), _p(dts), _p(zs), _p(A32)
    a.Bm, a.Cm = _p(Bt), _p(Ct)
    a.b_sb, a.b_sg, a.b_sn = g * nn, nn, 1
    a.c_sb, a.c_sg, a.c_sn = g * nn, nn, 1
    a.D, a.dt_bias, a.out = _p(D32), _p(b32), _p(out)
    _call(lib.ssm_selective_state_step, a)
    return out


# =========================================================================================
# ssd_chunk_scan (element-wise chunked recurrence)
# =========================================================================================


def _seq_lens(seq_meta: Optional[dict[str, Any]], nb: int, nl: int, device) -> Optional[Tensor]:
    """Per-row valid lengths as an int64 device tensor (reference.py:413-428)."""
    if not seq_meta:
        return None
    if seq_meta.get("cu_seqlens") is not None:
        cu = torch.as_tensor(seq_meta["cu_seqlens"]).to(device=device, dtype=torch.long)
        if cu.numel() != nb + 1:
            raise ValueError("cu_seqlens must have length B + 1.")
        return (cu[1:] - cu[:-1]).contiguous()
    if seq_meta.get("seq_lens") is not None:
        sl = torch.as_tensor(seq_meta["seq_lens"]).to(device=device, dtype=torch.long)
        if sl.numel() != nb:
            raise ValueError("seq_lens must have length B.")
        return sl.contiguous()
    raise ValueError("seq_meta must provide cu_seqlens or seq_lens.")


def _bc4(t: Optional[Tensor], kind: str) -> tuple[Optional[int], tuple[int, int, int, int]]:
    """Pointer and (sb, st, sh, sq) strides of a contiguous parameter of layout ``kind``."""
    if t is None:
        return None, (0, 0, 0, 0)
    if kind == "h":
        return t.data_ptr(), (0, 0, 1, 0)
    if kind == "hp":
        return t.data_ptr(), (0, 0, t.shape[1], 1)
    if kind == "bhp":
        return t.data_ptr(), (t.shape[1] * t.shape[2], 0, t.shape[2], 1)
    if kind == "blh":
        return t.data_ptr(), (t.shape[1] * t.shape[2], t.shape[2], 1, 0)
    if kind == "blhp":
        return t.data_ptr(), (t.shape[1] * t.shape[2] * t.shape[3], t.shape[2] * t.shape[3], t.shape[3], 1)
    raise AssertionError(kind)


def _set_bc4(dst: L.Bcast4, ptr: Optional[int], strides) -> None:
    dst.ptr = ptr
    dst.sb, dst.st, dst.sh, dst.sq = strides


class _ChunkCtx:
    def __init__(self, X, dt, A, B, C_, chunk_size, D, z, seq_meta, initial_states):
        if X.ndim != 4:
            raise ValueError("X must have shape (B, L, H, P).")
        if dt.ndim != 3:
            raise ValueError("dt must have shape (B, L, H).")
        nb, nl, nh, npj = X.shape
        if tuple(dt.shape) != (nb, nl, nh):
            raise ValueError("dt must align with (B, L, H).")
        if int(chunk_size) <= 0:
            raise ValueError("chunk_size must be positive.")
        _need_cuda(X, dt, A, B, C_, D, z, initial_states)
        self.shape = (nb, nl, nh, npj)
        self.chunk = int(chunk_size)
        self.io = _code(X, "ssd_chunk_scan")
        self.X, self.dt = _c(X), _c(dt.to(X.dtype))
        if A.ndim == 1:
            if A.shape[0] != nh:
                raise ValueError("A must have shape (H,) when 1-D.")
            self.A, self.kA = _f32(A), "h"
        elif A.ndim == 2:
            if tuple(A.shape) != (nh, npj):
                raise ValueError("A must have shape (H, P) when 2-D.")
            self.A, self.kA = _f32(A), "hp"
        else:
            raise ValueError("A must be 1-D or 2-D.")

        def coeff(name, p):
            if p.dim() == 2:
                if tuple(p.shape) != (nh, npj):
                    raise ValueError(f"{name} must have shape (H, P).")
                return "hp"
            if p.dim() == 3:
                if tuple(p.shape) != (nb, nh, npj):
                    raise ValueError(f"{name} must be (B, H, P) when 3-D.")
                return "bhp"
            if p.dim() == 4:
                if tuple(p.shape) != (nb, nl, nh, npj):
                    raise ValueError(f"{name} must have shape (B, L, H, P) when 4-D.")
                return "blhp"
            raise ValueError(f"Unsupported rank for {name}.")

        self.kB, self.kC = coeff("B", B), coeff("C", C_)
        self.kD = None
        if D is not None:
            if D.ndim == 1 and D.shape[0] == nh:
                self.kD = "h"
            elif D.ndim == 2 and tuple(D.shape) == (nh, npj):
                self.kD = "hp"
            else:
                raise ValueError("D must have shape (H,) or (H, P).")
        self.kz = None
        if z is not None:
            if z.ndim == 3 and tuple(z.shape) == (nb, nl, nh):
                self.kz = "blh"
            elif z.ndim == 4 and tuple(z.shape) == (nb, nl, nh, npj):
                self.kz = "blhp"
            else:
                raise ValueError("z must have shape (B, L, H) or (B, L, H, P).")
        if initial_states is not None and tuple(initial_states.shape) != (nb, nh, npj):
            raise ValueError("initial_states must have shape (B, H, P).")
        # B, C and z share one run-time dtype in the kernel
        par = [t for t in (B, C_, z) if t is not None]
        pd = X.dtype if all(t.dtype == X.dtype for t in par) else torch.float32  # the kernels take X's element type or fp32
        self.par = _CODES[pd]
        self.B, self.C = _c(B.to(pd)), _c(C_.to(pd))
        self.z = None if z is None else _c(z.to(pd))
        self.D = _f32(D)
        self.init = _f32(initial_states)
        self.lens = _seq_lens(seq_meta, nb, nl, X.device)

    def fill(self, a: L.ChunkArgs) -> None:
        nb, nl, nh, npj = self.shape
        a.batch, a.len, a.heads, a.proj = nb, nl, nh, npj
        a.io_dtype, a.par_dtype, a.chunk_size = self.io, self.par, self.chunk
        a.X, a.dt = _p(self.X), _p(self.dt)
        _set_bc4(a.A, *_bc4(self.A, self.kA))
        _set_bc4(a.Bm, *_bc4(self.B, self.kB))
        _set_bc4(a.Cm, *_bc4(self.C, self.kC))
        _set_bc4(a.D, *_bc4(self.D, self.kD or "h"))
        _set_bc4(a.z, *_bc4(self.z, self.kz or "blh"))
        _set_bc4(a.initial, *_bc4(self.init, "bhp"))
        a.seq_lens = _p(self.lens)


def _chunk_forward(cc: _ChunkCtx, want_final: bool = False):
    nb, nl, nh, npj = cc.shape
    lib = L.load()
    Y = torch.empty_like(cc.X)
    final = torch.empty(nb, nh, npj, dtype=torch.float32, device=cc.X.device) if want_final else None
    n = lib.ssm_chunk_scan_scratch_floats(nb, nl, nh, npj, cc.chunk)
    scratch = torch.empty(max(int(n), 1), dtype=torch.float32, device=cc.X.device)
    a = L.ChunkArgs()
    cc.fill(a)
    a.Y, a.final_state, a.scratch = _p(Y), _p(final), _p(scratch)
    _call(lib.ssm_chunk_scan_fwd, a)
    return Y, final


class _ChunkScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, dt, A, B, C_, chunk_size, D, z, seq_meta, initial_states):
        cc = _ChunkCtx(X, dt, A, B, C_, chunk_size, D, z, seq_meta, initial_states)
        Y, _ = _chunk_forward(cc)
        ctx.cc = cc
        ctx.like = (dt, A, B, C_, D, z, initial_states)
        _guard(ctx, X, dt, A, B, C_, D, z, initial_states)
        return Y

    @staticmethod
    def backward(ctx, gY):
        _check_guard(ctx)
        cc: _ChunkCtx = ctx.cc
        dt, A, B, C_, D, z, init = ctx.like
        nb, nl, nh, npj = cc.shape
        lib = L.load()
        dev = cc.X.device
        zeros = lambda t: None if t is None else torch.zeros(t.shape, dtype=torch.float32, device=dev)  # noqa: E731
        dX = torch.empty_like(cc.X)
        ddt = torch.zeros(nb, nl, nh, dtype=torch.float32, device=dev)
        # per-token B / C / z: their gradients are written by the kernel in the tensor's own type (no zero-fill, no fp32 copy)
        typed = [t is not None and k == "blhp" for t, k in ((cc.B, cc.kB), (cc.C, cc.kC), (cc.z, cc.kz))]
        own = lambda t, ty: torch.empty_like(t) if ty else zeros(t)  # noqa: E731
        dA, dB, dC, dD, dz, dI = zeros(cc.A), own(cc.B, typed[0]), own(cc.C, typed[1]), zeros(cc.D), own(cc.z, typed[2]), zeros(cc.init)
        hist = torch.empty(nb, max(nl, 1), nh, npj, dtype=torch.float32, device=dev)
        g = L.ChunkBwdArgs()
        cc.fill(g.fwd)
        g.fwd.typed_grads = sum(1 << i for i, ty in enumerate(typed) if ty)
        gy = _c(gY.to(cc.X.dtype))
        scratch = torch.empty(max(1, int(lib.ssm_chunk_scan_bwd_scratch_floats(nb, nl, nh, npj, cc.chunk))), dtype=torch.float32, device=dev)
        g.dY, g.dX, g.ddt, g.history, g.scratch = _p(gy), _p(dX), _p(ddt), _p(hist), _p(scratch)
        _set_bc4(g.dA, *_bc4(dA, cc.kA))
        _set_bc4(g.dB, *_bc4(dB, cc.kB))
        _set_bc4(g.dC, *_bc4(dC, cc.kC))
        _set_bc4(g.dD, *_bc4(dD, cc.kD or "h"))
        _set_bc4(g.dz, *_bc4(dz, cc.kz or "blh"))
        _set_bc4(g.dinitial, *_bc4(dI, "bhp"))
        _call(lib.ssm_chunk_scan_bwd, g)
        return (
            dX, ddt.to(dt.dtype), dA.to(A.dtype), dB.to(B.dtype), dC.to(C_.dtype), None,
            None if D is None else dD.to(D.dtype),
            None if z is None else dz.to(z.dtype),
            None,
            None if init is None else dI.to(init.dtype),
        )


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
    """Element-wise chunked recurrence over ``(B, L, H, P)`` (upstream ``ssm.ops.ssd_chunk_scan``,
    reference.py:312-463)."""
    if X.dtype == torch.float64:
        from . import ops_f64
        return ops_f64.ssd_chunk_scan(X, dt, A, B, C, chunk_size, D, z, seq_meta, initial_states)
    return _ChunkScanFn.apply(X, dt, A, B, C, chunk_size, D, z, seq_meta, initial_states)


# =========================================================================================
# dw_causal_conv
# =========================================================================================


class _ConvCtx:
    def __init__(self, x, weight, bias, activation, halo=None):
        if x.ndim != 3:
            raise ValueError("x must have shape (B, C, L) or (B, L, C).")
        nc = weight.shape[0]
        if x.shape[1] == nc:
            self.first = True
        elif x.shape[2] == nc:
            self.first = False
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
        act = str(activation).lower()
        if act not in ("silu", "swish", "identity", "none"):
            raise ValueError(f"Unsupported activation '{activation}'.")
        k = w2.shape[1]
        if k < 1 or k > 8:
            raise ValueError("dw_causal_conv: kernel width must be in [1, 8].")
        _need_cuda(x, weight, bias, halo)
        self.silu = act in ("silu", "swish")
        self.io = _code(x, "dw_causal_conv")
        self.x, self.w, self.b = (_rows(x) if self.first else _c(x)), _f32(w2), _f32(bias)
        self.nb = x.shape[0]
        self.nc, self.k = nc, k
        self.nl = x.shape[2] if self.first else x.shape[1]
        if halo is not None and tuple(halo.shape) != (self.nb, nc, k - 1):
            raise ValueError("halo must have shape (B, C, K-1).")
        self.halo = _f32(halo)

    def fill(self, a: L.ConvArgs) -> None:
        a.batch, a.channels, a.len, a.width = self.nb, self.nc, self.nl, self.k
        a.io_dtype, a.channels_first, a.silu = self.io, int(self.first), int(self.silu)
        a.x, a.weight, a.bias, a.halo = _p(self.x), _p(self.w), _p(self.b), _p(self.halo)
        if self.first and self.x.numel():
            a.row_sb, a.row_sc = self.x.stride(0), self.x.stride(1)
        else:
            a.row_sb, a.row_sc = self.nc * self.nl, self.nl


class _ConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, activation, halo):
        cc = _ConvCtx(x, weight, bias, activation, halo)
        y = torch.empty_like(cc.x)
        a = L.ConvArgs()
        cc.fill(a)
        a.y = _p(y)
        _call(L.load().ssm_dw_causal_conv_fwd, a)
        ctx.cc, ctx.like = cc, (weight, bias)
        _guard(ctx, x, weight, bias)
        return y

    @staticmethod
    def backward(ctx, gy):
        _check_guard(ctx)
        cc: _ConvCtx = ctx.cc
        weight, bias = ctx.like
        dev = cc.x.device
        dx = torch.empty_like(cc.x)
        dw = torch.zeros(cc.nc, cc.k, dtype=torch.float32, device=dev)
        db = torch.zeros(cc.nc, dtype=torch.float32, device=dev) if bias is not None else None
        g = L.ConvBwdArgs()
        cc.fill(g.fwd)
        go = _rows_like(gy, cc.x)
        g.dy, g.dx, g.dweight, g.dbias = _p(go), _p(dx), _p(dw), _p(db)
        _call(L.load().ssm_dw_causal_conv_bwd, g)
        return dx, dw.view(weight.shape).to(weight.dtype), None if bias is None else db.to(bias.dtype), None, None


def dw_causal_conv(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, activation: str = "silu",
                   halo: Optional[Tensor] = None) -> Tensor:
    """Depthwise causal conv1d with optional SiLU (upstream ``ssm.ops.dw_causal_conv``,
    reference.py:466-537).  Extension: ``halo`` ``(B, C, K-1)`` supplies the inputs that precede
    ``t = 0`` (sequence-sharded prefill) instead of zeros; no gradient flows into it."""
    if x.dtype == torch.float64:
        if halo is not None:
            raise ValueError("dw_causal_conv in float64 takes no halo.")
        from . import ops_f64
        return ops_f64.dw_causal_conv(x, weight, bias, activation)
    return _ConvFn.apply(x, weight, bias, activation, halo)


def dw_causal_conv_update(conv_state: Tensor, x: Tensor, weight: Tensor, bias: Optional[Tensor] = None,
                          activation: str = "silu") -> Tensor:
    """Extension: decode-time conv.  Rolls ``conv_state (B, C, K)`` (fp32, in place) left by one,
    appends ``x (B, C)`` and returns ``act(bias + <conv_state, weight>)`` (what upstream's
    ``Mamba1.step`` does with ``torch.roll``, modules/mamba1.py:345-353)."""
    if conv_state.ndim != 3 or x.ndim != 2 or conv_state.shape[:2] != x.shape:
        raise ValueError("conv_state must be (B, C, K) and x (B, C).")
    w2 = weight[:, 0, :] if weight.ndim == 3 else weight
    if tuple(w2.shape) != (x.shape[1], conv_state.shape[2]):
        raise ValueError("weight must have shape (C, K).")
    _need_cuda(conv_state, x, weight, bias)
    if conv_state.dtype != torch.float32 or not conv_state.is_contiguous():
        raise ValueError("conv_state must be a contiguous float32 tensor.")
    act = str(activation).lower()
    if act not in ("silu", "swish", "identity", "none"):
        raise ValueError(f"Unsupported activation '{activation}'.")
    xs, w32, b32 = _c(x), _f32(w2), _f32(bias)
    out = torch.empty_like(xs)
    a = L.ConvUpdateArgs()
    a.batch, a.channels, a.width, a.io_dtype = x.shape[0], x.shape[1], conv_state.shape[2], _code(x, "dw_causal_conv_update")
    a.silu = int(act in ("silu", "swish"))
    a.conv_state, a.x, a.weight, a.bias, a.out = _p(conv_state), _p(xs), _p(w32), _p(b32), _p(out)
    _call(L.load().ssm_dw_causal_conv_update, a)
    return out


# =========================================================================================
# fused_layer_norm
# =========================================================================================


class _NormCtx:
    def __init__(self, x, weight, bias, residual, is_rms, eps, prenorm):
        if x.ndim != 3:
            raise ValueError("x must have shape (B, L, D).")
        if tuple(weight.shape) != (x.shape[-1],):
            raise ValueError("weight must match the last dimension of x.")
        if bias is not None and tuple(bias.shape) != (x.shape[-1],):
            raise ValueError("bias must match the last dimension of x.")
        if residual is not None and residual.shape != x.shape:
            raise ValueError("residual must match the shape of x.")
        _need_cuda(x, weight, bias, residual)
        self.io = _code(x, "fused_layer_norm")
        self.x, self.w, self.b = _c(x), _f32(weight), _f32(bias)
        self.res = _c(residual)
        if self.res is not None:
            _code(self.res, "fused_layer_norm residual")
        self.is_rms, self.eps, self.prenorm = bool(is_rms), float(eps), bool(prenorm)

    def fill(self, a: L.NormArgs) -> None:
        a.rows, a.hidden = self.x.shape[0] * self.x.shape[1], self.x.shape[2]
        a.io_dtype = self.io
        a.res_dtype = _CODES[self.res.dtype] if self.res is not None else 0
        a.is_rms, a.prenorm, a.eps = int(self.is_rms), int(self.prenorm), self.eps
        a.x, a.residual, a.weight, a.bias = _p(self.x), _p(self.res), _p(self.w), _p(self.b)


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual, is_rms, eps, prenorm, return_residual, residual_dtype):
        nc = _NormCtx(x, weight, bias, residual, is_rms, eps, prenorm)
        y = torch.empty_like(nc.x)
        ro = torch.empty(nc.x.shape, dtype=residual_dtype, device=nc.x.device) if return_residual else None
        a = L.NormArgs()
        nc.fill(a)
        a.y, a.residual_out = _p(y), _p(ro)
        a.resout_dtype = _CODES[residual_dtype] if return_residual else 0
        _call(L.load().ssm_fused_add_norm_fwd, a)
        ctx.nc, ctx.like = nc, (weight, bias, residual)
        ctx.res_dtype = residual_dtype
        _guard(ctx, x, weight, bias, residual)
        if return_residual:
            return y, ro
        return y

    @staticmethod
    def backward(ctx, gy, gro=None):
        _check_guard(ctx)
        nc: _NormCtx = ctx.nc
        weight, bias, residual = ctx.like
        if gy is None:
            gy = torch.zeros_like(nc.x)
        lib = L.load()
        dev = nc.x.device
        hidden = nc.x.shape[2]
        rows = nc.x.shape[0] * nc.x.shape[1]
        dx = torch.empty_like(nc.x)
        dres = torch.empty_like(nc.res) if nc.res is not None else None
        dw = torch.empty(hidden, dtype=torch.float32, device=dev)
        db = torch.empty(hidden, dtype=torch.float32, device=dev) if bias is not None else None
        partial = torch.empty(int(lib.ssm_norm_bwd_scratch_floats(rows, hidden)), dtype=torch.float32, device=dev)
        g = L.NormBwdArgs()
        nc.fill(g.fwd)
        go = _c(gy.to(nc.x.dtype))
        g.dy, g.dx, g.dresidual, g.dweight, g.dbias, g.partial = _p(go), _p(dx), _p(dres), _p(dw), _p(db), _p(partial)
        gr = None
        if gro is not None:  # gradient arriving through the x + residual output: added to dx and dresidual inside the kernel
            gr = _c(gro.to(ctx.res_dtype))
            g.fwd.resout_dtype = _CODES[ctx.res_dtype]
            g.dresidual_out = _p(gr)
        _call(lib.ssm_fused_add_norm_bwd, g)
        return (
            dx, dw.to(weight.dtype), None if bias is None else db.to(bias.dtype),
            None if residual is None else dres.to(residual.dtype),
            None, None, None, None, None,
        )


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
    """Residual add fused with LayerNorm / RMSNorm (upstream ``ssm.ops.fused_layer_norm``,
    reference.py:540-609).  All arithmetic is fp32, which is what upstream does for fp32, bf16
    and fp16 inputs whatever ``residual_in_fp32`` says.  Extension: ``return_residual`` also
    returns ``x + residual`` (fp32 when ``residual_in_fp32``, else ``x.dtype``), the residual
    stream a stack of blocks passes on; gradients flow back through both outputs."""
    if x.dtype == torch.float64:
        from . import ops_f64
        return ops_f64.fused_layer_norm(x, weight, bias, residual, is_rms, eps, prenorm, residual_in_fp32, return_residual)
    rd = torch.float32 if residual_in_fp32 else x.dtype
    return _NormFn.apply(x, weight, bias, residual, is_rms, eps, prenorm, return_residual, rd)


# =========================================================================================
# ssd_scan: state-space-dual scan with a d_state axis (Mamba-2 layout)
# =========================================================================================


def _ssd_check(X, dt, A, B, C_, D, z, dt_bias, initial_states):
    if X.ndim != 4 or dt.ndim != 3:
        raise ValueError("X must be (B, L, H, P) and dt (B, L, H).")
    nb, nl, nh, npj = X.shape
    if tuple(dt.shape) != (nb, nl, nh):
        raise ValueError("dt must align with (B, L, H).")
    if tuple(A.shape) != (nh,):
        raise ValueError("A must have shape (H,).")
    if B.ndim != 4 or B.shape[0] != nb or B.shape[1] != nl or B.shape != C_.shape:
        raise ValueError("B and C must have shape (B, L, G, N).")
    ng, nn = B.shape[2], B.shape[3]
    if ng == 0 or nh % ng != 0:
        raise ValueError("Group dimension must divide H.")
    if D is not None and tuple(D.shape) not in ((nh,), (nh, npj)):
        raise ValueError("D must have shape (H,) or (H, P).")
    if z is not None and z.shape != X.shape:
        raise ValueError("z must have shape (B, L, H, P).")
    if dt_bias is not None and tuple(dt_bias.shape) != (nh,):
        raise ValueError("dt_bias must have shape (H,).")
    if initial_states is not None and tuple(initial_states.shape) != (nb, nh, npj, nn):
        raise ValueError("initial_states must have shape (B, H, P, N).")
    _need_cuda(X, dt, A, B, C_, D, z, dt_bias, initial_states)
    return nb, nl, nh, npj, ng, nn


def _ssd_via_scan(X, dt, A, B, C_, D, z, dt_bias, dt_softplus, initial_states):
    """The same recurrence through the selective-scan kernels on the ``H*P`` flattened channels
    (any shape and dtype the scan supports; differentiable).  Returns ``(Y, final_states fp32)``."""
    nb, nl, nh, npj = X.shape
    nn = B.shape[3]
    u = X.permute(0, 2, 3, 1).reshape(nb, nh * npj, nl)
    delta = dt.permute(0, 2, 1).repeat_interleave(npj, dim=1)
    A_full = A.float()[:, None, None].expand(nh, npj, nn).reshape(nh * npj, nn)
    Bs, Cs = B.permute(0, 2, 3, 1), C_.permute(0, 2, 3, 1)
    D_flat = None if D is None else (D.reshape(-1) if D.ndim == 2 else D[:, None].expand(nh, npj).reshape(-1))
    z_flat = None if z is None else z.permute(0, 2, 3, 1).reshape(nb, nh * npj, nl)
    b_flat = None if dt_bias is None else dt_bias[:, None].expand(nh, npj).reshape(-1)
    init = None if initial_states is None else initial_states.reshape(nb, nh * npj, nn)
    y, last = selective_scan(u, delta, A_full, Bs, Cs, D=D_flat, z=z_flat, dt_bias=b_flat, softplus=dt_softplus,
                             return_last_state=True, initial_state=init, keep_state_fp32=True)
    return y.reshape(nb, nh, npj, nl).permute(0, 3, 1, 2).contiguous(), last.reshape(nb, nh, npj, nn)


class _SsdWorkspace:
    """Scratch and bookkeeping of one tensor-core SSD call, kept so that a sequence shard can run
    the state phase, exchange states, and then finish from the same scratch."""

    def __init__(self, X, dt, A, B, C_, D, z, dt_bias, dt_softplus, chunk_size, dt_mode: int = 0, bc_width: int = 0, x_heads: int = 0):
        nb, nl, nh, npj = X.shape
        # x_heads: X holds only x_heads distinct input heads (head h reads input head h % x_heads); dt has one entry per head
        self.x_heads = int(x_heads)
        if x_heads:
            nh = dt.shape[2]
        # bc_width: B and C are stored bc_width (< d_state) wide and read as d_state-wide rows with zeros above
        self.bc_width = int(bc_width)
        self.shape = (nb, nl, nh, npj, B.shape[2], 2 * B.shape[3] if bc_width else B.shape[3])
        lib = L.load()
        io = X.dtype
        self.io, self.chunk, self.dt_mode = io, int(chunk_size), int(dt_mode)
        self.X, self.B, self.C = _c(X), _c(B.to(io)), _c(C_.to(io))
        # dt_mode 1 / 3: dt holds the fp32 step sizes as they are used (no bias, no softplus); 3 also gives the inputs unit weight
        self.dt = _c(dt.float()) if dt_mode else _c(dt.to(io))
        self.z = None if z is None else _c(z.to(io))
        self.A, self.D, self.bias = _f32(A), _f32(D), (None if dt_mode else _f32(dt_bias))
        self.d_has_p = int(D is not None and D.ndim == 2)
        self.softplus = int(bool(dt_softplus) and not dt_mode)
        self.nchunks = (nl + self.chunk - 1) // self.chunk
        self.ws = torch.empty(int(lib.ssm_ssd_scratch_bytes(nb, nl, nh)), dtype=torch.uint8, device=X.device)
        self._status = _DeviceStatus.of(X.device)
        self._status.poll()  # a wait that ran out in an earlier launch surfaces here, without a synchronisation
        self.status = self._status.word

    def run(self, phase: int, initial_states: Optional[Tensor], want_y: bool, row_dots: Optional[Tensor] = None,
            row_scale: Optional[Tensor] = None, keep_states_f32: bool = False):
        nb, nl, nh, npj, ng, nn = self.shape
        dev = self.X.device
        init32 = _f32(initial_states)
        Y = torch.empty(nb, nl, nh, npj, dtype=self.io, device=dev) if want_y else None
        final = torch.empty(nb, nh, npj, nn, dtype=torch.float32, device=dev)
        vec = nb * nh * self.nchunks * self.chunk * 4
        fin = int(L.load().ssm_ssd_state_scratch_bytes(nb, nl, nh))
        a = L.SsdArgs()
        a.batch, a.len, a.heads, a.headdim = nb, nl, nh, npj
        a.nstate, a.groups, a.chunk_size, a.io_dtype = nn, ng, self.chunk, _CODES[self.io]
        a.dt_softplus, a.d_has_p, a.phase, a.dt_mode = self.softplus, self.d_has_p, phase, self.dt_mode
        a.X, a.dt, a.A, a.Bm, a.Cm = _p(self.X), _p(self.dt), _p(self.A), _p(self.B), _p(self.C)
        a.D, a.z, a.dt_bias, a.initial_states = _p(self.D), _p(self.z), _p(self.bias), _p(init32)
        a.Y, a.final_states = _p(Y), _p(final)
        base = self.ws.data_ptr()
        a.ws_dt, a.ws_cum, a.ws_state, a.ws_state_in = base, base + vec, base + 2 * vec, base + 2 * vec + fin
        a.status = _p(self.status)
        a.row_dots = _p(row_dots)  # (B, L, H) fp32 zeros: z is then a dot-product partner, not a gate
        a.row_scale = _p(row_scale)  # (B, L, H) fp32 weights of the output rows
        a.bc_width = self.bc_width
        a.x_heads = self.x_heads
        self.states_f32 = None
        if keep_states_f32:  # (B, nchunks, H, P * N): the state before every chunk, unrounded
            self.states_f32 = torch.empty(nb, self.nchunks, nh, npj * nn, dtype=torch.float32, device=dev)
        a.ws_state_in_f32 = _p(self.states_f32)
        _call(L.load().ssm_ssd_fwd, a)
        self._status.after_launch()
        return Y, final

    def states_before_chunks(self) -> Tensor:
        """(B, nchunks, H, P * N) in the operand dtype: the state before every chunk as the last run left it in the
        scratch (element order of the scan kernel's operand tile, the same for every tile)."""
        nb, nl, nh, npj, _, nn = self.shape
        vec = nb * nh * self.nchunks * self.chunk * 4
        fin = int(L.load().ssm_ssd_state_scratch_bytes(nb, nl, nh))
        return self.ws[2 * vec + fin:].view(self.io).view(nb, self.nchunks, nh, npj * nn)

    def shard_summary(self) -> Tensor:
        """Flat fp32 view of what phase 1 left for the other ranks: the final state from a zero start, then (B, H) total log-decay."""
        nb, nl, nh, _, _, _ = self.shape
        vec = nb * nh * self.nchunks * self.chunk * 4
        n = int(L.load().ssm_ssd_shard_summary_floats(nb, nh))
        return self.ws[2 * vec: 2 * vec + n * 4].view(torch.float32)

    def total_log_decay(self) -> Tensor:
        """(B, H) sum over the shard of delta * A, read from the cumulative sums left in scratch."""
        nb, nl, nh, _, _, _ = self.shape
        vec = nb * nh * self.nchunks * self.chunk
        cum = self.ws[vec * 4: 2 * vec * 4].view(torch.float32).view(nb, nh, self.nchunks, self.chunk)
        return cum[..., -1].sum(-1) * math.log(2.0)  # the scratch holds base-2 exponents


def _ssd_tensor_core(X, dt, A, B, C_, D, z, dt_bias, dt_softplus, initial_states, chunk_size):
    w = _SsdWorkspace(X, dt, A, B, C_, D, z, dt_bias, dt_softplus, chunk_size)
    Y, final = w.run(0, initial_states, True)
    return Y, final, w.status


def ssd_tensor_core_supported(X: Tensor, B: Tensor, chunk_size: int) -> bool:
    """True when :func:`ssd_scan` runs on the tcgen05 kernels for these operands."""
    return bool(X.is_cuda and X.dtype in (torch.bfloat16, torch.float16)
                and L.load().ssm_ssd_supported(X.shape[3], B.shape[3], int(chunk_size), _CODES[X.dtype]))



def _ssd_dual_run(X, delta, A, B, C_, init, chunk, dt_mode, partner=None, row_scale=None, bc_width=0, keep_states_f32=False, x_heads=0):
    """One pass of the tensor-core kernels on ready-made fp32 step sizes; returns (Y, final_states, workspace, dots).
    With ``partner (B, L, H, P)`` the pass also returns ``dots[b, t, h] = sum_p y[p] partner[p]`` from the fp32 accumulators."""
    w = _SsdWorkspace(X, delta, A, B, C_, None, partner, None, False, chunk, dt_mode=dt_mode, bc_width=bc_width, x_heads=x_heads)
    dots = None if partner is None else torch.zeros(delta.shape[:3], dtype=torch.float32, device=X.device)
    Y, final = w.run(0, init, True, row_dots=dots, row_scale=None if row_scale is None else _c(row_scale.float()),
                     keep_states_f32=keep_states_f32)
    return Y, final, w, dots


def _time_flip(t: Tensor, length: int) -> Tensor:
    """``out[b, length - 1 - i] = t[b, i]`` for a contiguous ``(B, L, ...)`` tensor with ``L <= length``; rows beyond ``L`` are zero."""
    t = _c(t)
    out = torch.empty((t.shape[0], length, *t.shape[2:]), dtype=t.dtype, device=t.device)
    row = t[0, 0].numel() * t.element_size() if t.shape[1] else 0
    L.check(L.load().ssm_time_flip(_p(t), _p(out), t.shape[0], length, t.shape[1], row, _stream()))
    return out


def _ssd_backward_dual(X, dt, A, B, C_, D, z, dt_bias, dt_softplus, init, chunk, gY, gfinal):
    """Gradients of the state-space-dual scan in the dual (chunked GEMM) form, every contraction on the tcgen05 kernels
    of the forward pass.  With ``a_t = delta_t A`` and the adjoint state ``G_t = C_t dy_t^T + exp(a_{t+1}) G_{t+1}``:

    * ``d(delta x)_t = G_t B_t`` is the forward recurrence run on the time-reversed sequence with ``B`` and ``C``
      exchanged, ``dy`` as the input, unit input weight and the decays shifted by one step; its final state is the
      gradient of the initial state (up to the first decay);
    * ``dC_t = S_t dy_t`` (and ``dB_t = delta_t G_t x_t`` on the reversed sequence) is the same recurrence with the roles
      of the head and state axes exchanged: per head, ``x`` and ``dy`` take the places of ``B`` and ``C`` (64 wide, read as
      128 with zeros above) and the two halves of ``B`` are the inputs of two heads of 64;
    * the gradient of the decay exponent obeys ``da_{t+1} = da_t + d(delta x)_t . (delta x)_t - dy_t . y_t`` (``y`` without
      the skip term); the running sum restarts at every chunk from ``<G, S>`` of the two passes' chunk states.  The
      adjoint pass weights its rows by ``delta`` so that it rounds the same masked tiles as the forward pass; the two
      dot products come from the passes' fp32 accumulators.

    The passes over ``(B, L, H, P)`` around the four runs are the kernels of ``csrc/ssd_bwd.cu``; only ``(B, L, H)``-sized
    bookkeeping of the step sizes is PyTorch.  Returns the nine gradients."""
    lib = L.load()
    nb, nl, nh, npj = X.shape
    ng, nn = B.shape[2], B.shape[3]
    rep = nh // ng
    io, dev = X.dtype, X.device
    code = _CODES[io]
    f32 = torch.float32
    A32 = A.float()
    pre_act = dt.float() if dt_bias is None else dt.float() + dt_bias.float()
    delta = F.softplus(pre_act) if dt_softplus else pre_act
    pad = (-nl) % chunk  # whole chunks, so that the chunks of the reversed sequence are the chunks of the forward one
    lp = nl + pad
    nchunks = lp // chunk
    Xc, Bc, Cc = _c(X), _c(B.to(io)), _c(C_.to(io))
    zc = None if z is None else _c(z.to(io))
    gy = torch.zeros_like(Xc) if gY is None else _c(gY.to(io))
    D32 = _f32(D)
    if pad:
        delta = F.pad(delta, (0, 0, 0, pad))
        Xp, Bp, Cp = F.pad(Xc, (0, 0, 0, 0, 0, pad)), F.pad(Bc, (0, 0, 0, 0, 0, pad)), F.pad(Cc, (0, 0, 0, 0, 0, pad))
    else:
        delta, Xp, Bp, Cp = _c(delta), Xc, Bc, Cc
    # dy = gY silu(z), in time order and reversed
    dy = torch.empty(nb, lp, nh, npj, dtype=io, device=dev)
    dy_r = torch.empty_like(dy)
    g = L.SsdBwdArgs()
    g.batch, g.len, g.len_valid, g.heads, g.headdim, g.io_dtype = nb, lp, nl, nh, npj, code
    g.d_has_p = int(D is not None and D.ndim == 2)
    g.gY, g.z, g.dy, g.dy_rev = _p(gy), _p(zc), _p(dy), _p(dy_r)
    _call(lib.ssm_ssd_bwd_gate, g)
    # (1) forward again without skip and gate: y, dy . y, and the state before every chunk
    y_plain, _, w_fwd, u = _ssd_dual_run(Xp, delta, A32, Bp, Cp, init, chunk, 1, partner=dy, keep_states_f32=True)
    # (2) adjoint recurrence on the reversed sequence, rows weighted by delta of the source step: the output is the x
    # gradient without the skip term, and the masked tiles round exactly like those of pass (1), which lets (4) telescope
    X_r, B_r, C_r = _time_flip(Xc, lp), _time_flip(Bc, lp), _time_flip(Cc, lp)
    delta_r = torch.zeros_like(delta)
    delta_r[:, 1:] = delta.flip(1)[:, :-1]
    g_init = None if gfinal is None else gfinal.float()
    dx_r, fin_r, w_adj, qd_r = _ssd_dual_run(dy_r, delta_r, A32, C_r, B_r, g_init, chunk, 3, partner=X_r, row_scale=delta.flip(1),
                                                keep_states_f32=True)
    dinit = torch.exp(delta[:, 0] * A32)[..., None, None] * fin_r
    # dz, dX (+ D dy), dD
    dX = torch.empty_like(Xc)
    dz = None if zc is None else torch.empty_like(zc)
    dD = None if D is None else torch.zeros(D.shape, dtype=f32, device=dev)
    g.X, g.y_plain, g.dx_rev, g.D, g.dX, g.dz, g.dD = _p(Xc), _p(y_plain), _p(dx_r), _p(D32), _p(dX), _p(dz), _p(dD)
    _call(lib.ssm_ssd_bwd_finish, g)
    del y_plain, dx_r

    # (3) dC and dB: head and state axes exchanged, one group per head, the halves of B (C) as the inputs of two heads
    # With a single group the halves are not written out per head: the kernels read input head h % 2 (x_heads = 2).
    xh2 = 2 if (ng == 1 and rep > 1) else 0

    def halves(t):  # (B, L, G, N) -> (B, L, 2 H, N / 2): every head gets its group's row, the two halves as two heads
        if rep == 1 or xh2:
            return t.reshape(nb, lp, 2 * ng, nn // 2)
        out = torch.empty(nb, lp, 2 * nh, nn // 2, dtype=io, device=dev)
        L.check(lib.ssm_ssd_bwd_spread(_p(t), _p(out), nb * lp, nh, ng, nn * t.element_size(), _stream()))
        return out

    def state_t(s):  # (B, H, P, N) fp32 -> (B, 2 H, N / 2, N): transposed, the P axis zero-padded to N
        return None if s is None else F.pad(s.float().transpose(2, 3).reshape(nb, 2 * nh, nn // 2, npj), (0, nn - npj))

    def group_sum(y, weight, reversed_, like):
        out_dtype = io if like.dtype == io else f32
        out = torch.empty(nb, nl, ng, nn, dtype=out_dtype, device=dev)
        L.check(lib.ssm_ssd_bwd_group_sum(_p(y), _p(weight), _p(out), nb, lp, nl, nh, ng, nn, int(reversed_), code, _CODES[out_dtype], _stream()))
        return out

    A2 = A32.repeat_interleave(2)
    yc = _ssd_dual_run(halves(Bp), delta.repeat_interleave(2, 2), A2, Xp, dy, state_t(init), chunk, 1 | 4, bc_width=npj, x_heads=xh2)[0]
    dC = group_sum(yc, None, False, C_)
    del yc
    yb = _ssd_dual_run(halves(C_r), delta_r.repeat_interleave(2, 2), A2, dy_r, X_r, state_t(g_init), chunk, 3 | 4, bc_width=npj, x_heads=xh2)[0]
    dB = group_sum(yb, delta, True, B)
    del yb
    # (4) decay exponent: chunk-local running sums started from <adjoint state, state> at the chunk boundaries
    qd = qd_r.flip(1)  # (B, L, H): delta_t d(delta x)_t . x_t
    q = torch.where(delta > 0, qd / delta, torch.zeros_like(qd))
    r = qd - u
    start = torch.empty(nb, nchunks, nh, dtype=f32, device=dev)
    L.check(lib.ssm_ssd_state_dot(_p(w_fwd.states_f32), _p(w_adj.states_f32), _p(start), nb, nchunks, nh, npj * nn, _CODES[f32], _stream()))
    if nchunks > 1:
        start[:, 1:] *= torch.exp(delta[:, chunk::chunk] * A32)  # decay of the first step of chunks 1 ..
    if init is not None:
        start[:, 0] = (dinit * init.float()).sum((-1, -2))
    rc = r.view(nb, nchunks, chunk, nh)
    da = (start[:, :, None] + torch.cumsum(rc, 2) - rc).reshape(nb, lp, nh)
    ddelta = (q + A32 * da)[:, :nl]
    dA = (delta * da).sum((0, 1))
    if dt_softplus:
        ddelta = ddelta * torch.sigmoid(pre_act)
    dbias = None if dt_bias is None else ddelta.sum((0, 1))
    return dX, ddelta, dA, dB, dC, dD, dz, dbias, dinit


class _SsdFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, dt, A, B, C_, D, z, dt_bias, dt_softplus, initial_states, chunk_size, check_status, dual_backward):
        _ssd_check(X, dt, A, B, C_, D, z, dt_bias, initial_states)
        ctx.args = (X, dt, A, B, C_, D, z, dt_bias, dt_softplus, initial_states)
        _guard(ctx, X, dt, A, B, C_, D, z, dt_bias, initial_states)
        ctx.chunk = int(chunk_size)
        ctx.dual = bool(dual_backward) and ssd_tensor_core_supported(X, B, chunk_size)
        if ssd_tensor_core_supported(X, B, chunk_size):
            Y, final, _ = _ssd_tensor_core(X, dt, A, B, C_, D, z, dt_bias, dt_softplus, initial_states, int(chunk_size))
            if check_status:
                ssd_check_status(X.device)
            return Y, final
        with torch.no_grad():
            return _ssd_via_scan(X, dt, A, B, C_, D, z, dt_bias, dt_softplus, initial_states)

    @staticmethod
    def backward(ctx, gY, gfinal):
        _check_guard(ctx)
        X, dt, A, B, C_, D, z, dt_bias, dt_softplus, init = ctx.args
        if ctx.dual:
            with torch.no_grad():
                grads = _ssd_backward_dual(X, dt, A, B, C_, D, z, dt_bias, dt_softplus, init, ctx.chunk, gY, gfinal)
            srcs = (X, dt, A, B, C_, D, z, dt_bias, init)
            res = [None if (t is None or g is None or not t.requires_grad) else g.to(t.dtype).reshape(t.shape) for t, g in zip(srcs, grads)]
            return (*res[:8], None, res[8], None, None, None)
        leaves = [None if t is None else t.detach().requires_grad_(t.requires_grad) for t in (X, dt, A, B, C_, D, z, dt_bias, init)]
        with torch.enable_grad():
            Y, final = _ssd_via_scan(*leaves[:8], dt_softplus, leaves[8])
        live = [t for t in leaves if t is not None and t.requires_grad]
        outs, gouts = [Y], [gY if gY is not None else torch.zeros_like(Y)]
        if gfinal is not None:
            outs.append(final)
            gouts.append(gfinal)
        grads = iter(torch.autograd.grad(outs, live, gouts, allow_unused=True))
        res = [next(grads) if (t is not None and t.requires_grad) else None for t in leaves]
        return (*res[:8], None, res[8], None, None, None)


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
    check_status: bool = False,
    backward: str = "dual",
    cu_seqlens: Optional[Tensor] = None,
    seq_reset: bool = True,
    return_varlen_states: bool = False,
):
    """Extension: state-space-dual scan with a ``d_state`` axis (Mamba-2 layout).

    ``X (B,L,H,P)``, ``dt (B,L,H)``, ``A (H,)``, ``B/C (B,L,G,N)``, ``D (H,)|(H,P)``, ``z (B,L,H,P)``,
    state ``(B,H,P,N)`` fp32.  It is upstream's ``selective_scan`` recurrence (reference.py:173-188)
    on channel ``h*P+p`` with per-head ``dt`` and ``A``.  For headdim 64, d_state 128, chunk 256 and
    bf16 / fp16 operands the forward runs as chunked GEMMs on the tcgen05 tensor cores, and so does the
    backward (``backward="dual"``: four more runs of the same kernels on transformed operands; its
    gradients carry the rounding of 16-bit operands, about 0.3 % of each contraction).  ``cu_seqlens (S + 1,)``
    marks ``S`` sequences packed along ``L`` of a batch of one: ``return_varlen_states`` adds the state after the last
    token of every sequence ``(S, H, P, N)``, each scanned from zero, and with ``seq_reset`` (default) ``Y`` restarts at
    every boundary too (without it ``Y`` runs through, as upstream mamba-ssm does when given no ``seq_idx``).  Any other shape or
    dtype, and ``backward="scan"``, goes through the selective-scan kernels on the flattened channels
    (fp32 arithmetic, an order of magnitude slower at these shapes).  A bounded device-side wait that runs out (it never should) is reported by the next
    ``ssd_scan`` call on the device, or at once by ``check_status=True`` / :func:`ssd_check_status`, which synchronise.
    """
    if backward not in ("dual", "scan"):
        raise ValueError('backward must be "dual" or "scan".')
    dual = backward == "dual"
    if cu_seqlens is None:
        if return_varlen_states:
            raise ValueError("return_varlen_states needs cu_seqlens.")
        Y, final = _SsdFn.apply(X, dt, A, B, C, D, z, dt_bias, dt_softplus, initial_states, chunk_size, check_status, dual)
        return (Y, final) if return_final_states else Y
    # packed sequences: every sequence is its own scan from a zero state (chunks counted from its first token), so the
    # kernels see plain dense problems; the boundaries are host integers (one read of cu_seqlens)
    if X.ndim != 4 or X.shape[0] != 1:
        raise ValueError("cu_seqlens needs a batch of one (sequences packed along L).")
    if initial_states is not None and seq_reset:
        raise ValueError("initial_states cannot be combined with sequences that restart at cu_seqlens.")
    cu = [int(v) for v in torch.as_tensor(cu_seqlens).tolist()]
    if len(cu) < 2 or cu[0] != 0 or cu[-1] != X.shape[1] or any(b < a for a, b in zip(cu, cu[1:])):
        raise ValueError("cu_seqlens must rise from 0 to L.")
    cut = lambda t, a, b: None if t is None else t[:, a:b]  # noqa: E731
    parts, states = [], []
    for a, b in zip(cu, cu[1:]):
        if b == a:
            states.append(torch.zeros(X.shape[2], X.shape[3], B.shape[3], dtype=torch.float32, device=X.device))
            continue
        y_k, s_k = _SsdFn.apply(cut(X, a, b), cut(dt, a, b), A, cut(B, a, b), cut(C, a, b), D, cut(z, a, b), dt_bias, dt_softplus, None,
                                chunk_size, check_status, dual)
        parts.append(y_k)
        states.append(s_k[0])
    varlen = torch.stack(states)
    if seq_reset:
        Y, final = (torch.cat(parts, 1) if parts else torch.empty_like(X)), varlen[-1:].clone()
    else:  # upstream mamba-ssm given cu_seqlens without seq_idx: Y runs through the boundaries, only the states are per sequence
        Y, final = _SsdFn.apply(X, dt, A, B, C, D, z, dt_bias, dt_softplus, initial_states, chunk_size, check_status, dual)
    out = [Y]
    if return_final_states:
        out.append(final)
    if return_varlen_states:
        out.append(varlen)
    return out[0] if len(out) == 1 else tuple(out)


__all__ = [
    "selective_scan",
    "selective_state_step",
    "selective_state_step_heads",
    "ssd_chunk_scan",
    "dw_causal_conv",
    "dw_causal_conv_update",
    "fused_layer_norm",
    "ssd_scan",
    "ssd_check_status",
    "ssd_wait_selftest",
    "ssd_tensor_core_supported",
]
