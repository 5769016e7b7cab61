"""Sequence-sharded state-space-dual scan across GPUs (one process per GPU, ``torch.distributed``).

The reference package has no distributed code at all; this is the multi-GPU form of the SSD hot
path.  Rank ``r`` of ``R`` holds the contiguous tokens ``[r L/R, (r+1) L/R)`` of every sequence.
The recurrence is linear in the state, so a shard acts on it as ``S_out = P * S_in + S_loc`` with
``P = exp(sum_t delta_t A)`` per head and ``S_loc`` its final state from a zero start.  Each rank

1. runs the state phase on its shard (no output yet),
2. all-gathers ``(S_loc, log P)`` -- ``batch x heads x headdim x d_state`` fp32 per rank over
   NCCL / NVLink -- and folds the shards before it into its true incoming state (the fold is
   associative, so there is no serial hand-off chain),
3. finishes from the scratch of step 1 with that incoming state and produces its slice of ``Y``.

Received data always lands in this GPU's own memory through NCCL before any kernel reads it.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

Tensor = torch.Tensor


def fold_incoming_state(states: Tensor, log_decay: Tensor, rank: int, initial: Optional[Tensor] = None) -> Tensor:
    """Incoming state of shard ``rank``.

    ``states``: ``R`` tensors ``(B, H, P, N)``, every shard's final state from a zero start; ``log_decay``: ``R`` tensors ``(B, H)``,
    every shard's total ``sum delta A``.  ``initial`` is the state before shard 0.
    ``S_in[r] = sum_{q<r} exp(sum_{q<m<r} logP_m) S_q  (+ exp(sum_{m<r} logP_m) initial)``.
    """
    if rank == 0:
        return torch.zeros_like(states[0]) if initial is None else initial.to(states[0].dtype).clone()
    # weight of shard q's state (and of the initial state) at the start of shard `rank`: the decay of the shards in between
    logs = torch.stack([log_decay[q] for q in range(rank)])                                   # (rank, B, H)
    after = torch.flip(torch.cumsum(torch.flip(logs, [0]), 0), [0]) - logs                    # sum over q < m < rank
    s = (torch.stack([states[q] for q in range(rank)]) * torch.exp(after)[..., None, None]).sum(0)
    if initial is not None:
        s = s + torch.exp(logs.sum(0))[..., None, None] * initial.to(s.dtype)
    return s


def outgoing_state(incoming: Tensor, local: Tensor, log_decay: Tensor) -> Tensor:
    """Final state of a shard given its incoming state."""
    return torch.exp(log_decay)[..., None, None] * incoming + local


def ssd_scan_sequence_parallel(
    state_phase: Callable[[], tuple[Tensor, Tensor]],
    finish_phase: Callable[[Tensor], tuple[Tensor, Tensor]],
    group: Optional[dist.ProcessGroup] = None,
    initial_states: Optional[Tensor] = None,
):
    """Generic driver: ``state_phase() -> (S_loc, logP)``; ``finish_phase(S_in) -> (Y, S_out)``.
    Returns ``(Y_shard, S_out)`` where ``S_out`` on the last rank is the sequence's final state."""
    alone = not (dist.is_available() and dist.is_initialized())
    rank, world = (0, 1) if alone else (dist.get_rank(group), dist.get_world_size(group))
    s_loc, logp = state_phase()
    if world == 1:
        return finish_phase(None if initial_states is None else initial_states.to(s_loc.dtype))
    # one message per rank: the state with its log-decay appended
    nbh = logp.numel()
    packed = torch.cat([s_loc.reshape(nbh, -1), logp.reshape(nbh, 1).to(s_loc.dtype)], dim=1).contiguous()
    gathered = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(gathered, packed, group=group)
    if rank == 0:
        return finish_phase(None if initial_states is None else initial_states.to(s_loc.dtype))
    all_s = [gk[:, :-1].reshape(s_loc.shape) for gk in gathered[:rank]]
    all_p = [gk[:, -1].reshape(logp.shape) for gk in gathered[:rank]]
    s_in = fold_incoming_state(all_s, all_p, rank, initial_states)
    return finish_phase(s_in)


def ssd_scan_sharded(X, dt, A, B, C, chunk_size=256, D=None, z=None, dt_bias=None, dt_softplus=False,
                     initial_states=None, group=None):
    """Sequence-parallel :func:`ssm_b200.ops.ssd_scan` on this rank's shard (tensor-core path).

    ``z`` may be a zero-argument callable that returns the gate: it is called once the exchange of the shard states has
    been posted, so the work that produces the gate (a projection GEMM) runs while the ranks wait for one another."""
    from . import ops
    z_fn = z if callable(z) else None
    if z_fn is not None:
        z = None

    if not ops.ssd_tensor_core_supported(X, B, chunk_size):
        raise ValueError("ssd_scan_sharded needs the tensor-core shape (headdim 64, d_state 128, chunk 256, bf16/fp16)")
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (X, dt, A, B, C, D, z, dt_bias, initial_states)):
        raise RuntimeError("ssd_scan_sharded is forward-only: call it under torch.no_grad() (its outputs carry no autograd history)")
    ops._ssd_check(X, dt, A, B, C, D, z, dt_bias, None)
    w = ops._SsdWorkspace(X, dt, A, B, C, D, z, dt_bias, dt_softplus, chunk_size)

    def resolve_gate():
        if z_fn is None:
            return
        gate = z_fn()
        if gate is not None:
            if tuple(gate.shape) != tuple(X.shape):
                raise ValueError("z must have the shape of X.")
            w.z = gate.to(w.io).contiguous()

    def state_phase():
        _, s_loc = w.run(1, None, False)
        return s_loc, w.total_log_decay()

    def finish_phase(s_in):
        return w.run(2, s_in, True)

    alone = not (dist.is_available() and dist.is_initialized())
    world = 1 if alone else dist.get_world_size(group)
    if world > 1 and dist.get_backend(group) == "nccl":
        # fast path: the summary phase 1 leaves in the scratch is gathered as it is and folded by one kernel
        from . import _lib as L

        rank = dist.get_rank(group)
        w.run(1, None, False)
        mine = w.shard_summary()
        gathered = torch.empty(world * mine.numel(), dtype=torch.float32, device=mine.device)
        work = dist.all_gather_into_tensor(gathered, mine, group=group, async_op=True)
        resolve_gate()  # enqueued behind phase 1 on this stream, beside the gather on the communicator's
        work.wait()
        if rank == 0 and initial_states is None:
            return finish_phase(None)
        nb, _, nh, npj, _, nn = w.shape
        s_in = torch.empty(nb, nh, npj, nn, dtype=torch.float32, device=mine.device)
        init = None if initial_states is None else initial_states.to(torch.float32).contiguous()
        L.check(L.load().ssm_ssd_fold_shards(gathered.data_ptr(), world, rank, nb, nh, None if init is None else init.data_ptr(), s_in.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream))
        return finish_phase(s_in)
    resolve_gate()
    return ssd_scan_sequence_parallel(state_phase, finish_phase, group, initial_states)


def exchange_conv_halo(x_shard: Tensor, width: int, group=None, channels_first: bool = True, _defer: Optional[list] = None) -> Optional[Tensor]:
    """Send this shard's last ``width-1`` inputs to the next rank; returns the halo ``(B, C, width-1)``
    fp32 received from the previous rank (``None`` on rank 0), for ``dw_causal_conv(..., halo=)``."""
    alone = not (dist.is_available() and dist.is_initialized())
    rank, world = (0, 1) if alone else (dist.get_rank(group), dist.get_world_size(group))
    k = width - 1
    if k == 0 or world == 1:
        return None
    tail = (x_shard[:, :, -k:] if channels_first else x_shard[:, -k:, :].transpose(1, 2)).float().contiguous()
    recv = torch.empty_like(tail)
    ops_ = []
    if rank + 1 < world:
        ops_.append(dist.P2POp(dist.isend, tail, dist.get_global_rank(group, rank + 1) if group else rank + 1, group))
    if rank > 0:
        ops_.append(dist.P2POp(dist.irecv, recv, dist.get_global_rank(group, rank - 1) if group else rank - 1, group))
    reqs = dist.batch_isend_irecv(ops_)
    if _defer is not None:  # the caller waits later (post_conv_halos)
        _defer.extend(reqs)
        _defer.append(tail)  # the message stays alive until then
        return recv if rank > 0 else None
    for req in reqs:
        req.wait()
    return recv if rank > 0 else None


class PostedHalos:
    """The conv halos of a shard on their way (see :func:`post_conv_halos`); ``wait()`` returns them."""

    def __init__(self, widths, halo, pending):
        self._widths, self._halo, self._pending = widths, halo, pending

    def wait(self):
        for req in self._pending:
            if hasattr(req, "wait"):
                req.wait()
        self._pending = []
        if self._halo is None:
            return [None for _ in self._widths]
        out, c0 = [], 0
        for c in self._widths:
            out.append(self._halo[:, c0:c0 + c, :].contiguous())
            c0 += c
        return out


def post_conv_halos(parts, width: int, group=None) -> PostedHalos:
    """Posts the exchange of :func:`exchange_conv_halos` and returns without waiting for it: what the caller enqueues
    before ``wait()`` (projections that do not need the halo) runs while the message travels."""
    alone = not (dist.is_available() and dist.is_initialized())
    world = 1 if alone else dist.get_world_size(group)
    widths = [p.shape[-1] for p in parts]
    if width <= 1 or world == 1:
        return PostedHalos(widths, None, [])
    joined = torch.cat([p[:, -(width - 1):, :] for p in parts], dim=-1)  # (B, K-1, sum C_i)
    pending: list = []
    halo = exchange_conv_halo(joined, width, group, channels_first=False, _defer=pending)
    return PostedHalos(widths, halo, pending)


def exchange_conv_halos(parts, width: int, group=None):
    """One exchange for several channels-last conv inputs ``(B, L, C_i)`` of the same shard: their last
    ``width-1`` tokens travel to the next rank as one message.  Returns one halo ``(B, C_i, width-1)`` per
    part (fp32), or ``None`` for each on rank 0 / without a process group."""
    return post_conv_halos(parts, width, group).wait()
