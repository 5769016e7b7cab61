"""Sequence-parallel hand-off logic on CPU ranks (gloo, world size 2 and 3): the shard fold and
the two-phase driver, with the CPU oracle standing in for the per-shard kernels."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ssm_oracle as orc


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make(seed, nb, nl, nh, npj, ng, nn):
    g = torch.Generator().manual_seed(seed)
    return dict(
        X=torch.randn(nb, nl, nh, npj, generator=g), dt=torch.rand(nb, nl, nh, generator=g) * 0.3 + 0.01,
        A=-torch.exp(torch.rand(nh, generator=g)), B=torch.randn(nb, nl, ng, nn, generator=g) / nn ** 0.5,
        C=torch.randn(nb, nl, ng, nn, generator=g) / nn ** 0.5, D=torch.randn(nh, generator=g),
        z=torch.randn(nb, nl, nh, npj, generator=g), init=torch.randn(nb, nh, npj, nn, generator=g) * 0.3)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ssm_b200 import seqpar

        torch.set_num_threads(1)
        nb, nl, nh, npj, ng, nn = 2, 60, 3, 4, 1, 8
        t = _make(0, nb, nl, nh, npj, ng, nn)
        per = nl // world
        sl = slice(rank * per, (rank + 1) * per)
        loc = {k: (v[:, sl] if k in ("X", "dt", "B", "C", "z") else v) for k, v in t.items()}

        def state_phase():
            _, s = orc.ssd_scan(loc["X"], loc["dt"], loc["A"], loc["B"], loc["C"], 16, return_final_states=True)
            return s, (loc["dt"] * loc["A"][None, None]).sum(1)

        def finish_phase(s_in):
            return orc.ssd_scan(loc["X"], loc["dt"], loc["A"], loc["B"], loc["C"], 16, D=loc["D"], z=loc["z"], initial_states=s_in,
                                return_final_states=True)

        Y, S = seqpar.ssd_scan_sequence_parallel(state_phase, finish_phase, None, t["init"])
        Yf, Sf = orc.ssd_scan(t["X"], t["dt"], t["A"], t["B"], t["C"], 16, D=t["D"], z=t["z"], initial_states=t["init"],
                              return_final_states=True)
        torch.testing.assert_close(Y, Yf[:, sl], rtol=1e-4, atol=1e-5)
        if rank == world - 1:
            torch.testing.assert_close(S, Sf, rtol=1e-4, atol=1e-5)
        # conv halo: shards with the received halo reproduce the unsharded convolution
        x = torch.randn(2, 5, 24, generator=torch.Generator().manual_seed(1))
        w = torch.rand(5, 4, generator=torch.Generator().manual_seed(2)) - 0.5
        xs = x[:, :, rank * (24 // world):(rank + 1) * (24 // world)].contiguous()
        halo = seqpar.exchange_conv_halo(xs, 4)
        assert (halo is None) == (rank == 0)
        full = orc.dw_causal_conv(x, w, None, "silu")
        xs_ext = xs if halo is None else torch.cat([halo, xs], dim=-1)
        got = orc.dw_causal_conv(xs_ext, w, None, "silu")[:, :, -xs.shape[-1]:]
        torch.testing.assert_close(got, full[:, :, rank * (24 // world):(rank + 1) * (24 // world)], rtol=1e-5, atol=1e-6)
        # several channels-last inputs in one message, posted first and awaited after other work was enqueued
        parts = [xs.transpose(1, 2).contiguous(), (2.0 * xs[:, :2]).transpose(1, 2).contiguous()]  # (B, L, 5) and (B, L, 2)
        posted = seqpar.post_conv_halos(parts, 4)
        busy = (parts[0] @ torch.ones(5, 3)).sum()  # stands for the projection that runs while the message travels
        halos = posted.wait()
        assert torch.isfinite(busy)
        if rank == 0:
            assert halos == [None, None]
        else:
            torch.testing.assert_close(halos[0], halo)
            torch.testing.assert_close(halos[1], 2.0 * halo[:, :2])
        assert [None if h is None else tuple(h.shape) for h in seqpar.exchange_conv_halos(parts, 4)] == \
            [None if h is None else tuple(h.shape) for h in halos]
        out.put((rank, "ok"))
    except Exception as exc:  # noqa: BLE001
        out.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_parallel_handoff_on_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, "ok") for r in range(world)], res


def test_fold_matches_sequential_chain():
    from ssm_b200 import seqpar

    g = torch.Generator().manual_seed(3)
    R, nb, nh = 4, 2, 3
    states = torch.randn(R, nb, nh, 2, 5, generator=g)
    logp = -torch.rand(R, nb, nh, generator=g)
    init = torch.randn(nb, nh, 2, 5, generator=g)
    s = init.clone()
    for r in range(R):
        torch.testing.assert_close(seqpar.fold_incoming_state(states, logp, r, init), s)
        s = seqpar.outgoing_state(s, states[r], logp[r])


def _failing_worker(rank, world, port, out):
    """Rank 1 raises before it joins the hand-off; the others must come back with an error instead of waiting forever."""
    import datetime

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        from ssm_b200 import seqpar

        torch.set_num_threads(1)
        nb, nh, npj, nn = 1, 2, 4, 8

        def state_phase():
            if rank == 1:
                raise ValueError("injected failure on rank 1 before the hand-off")
            return torch.ones(nb, nh, npj, nn), torch.zeros(nb, nh)

        def finish_phase(s_in):
            return torch.zeros(nb, 4, nh, npj), torch.ones(nb, nh, npj, nn)

        seqpar.ssd_scan_sequence_parallel(state_phase, finish_phase, None, None)
        out.put((rank, "completed"))
    except ValueError as exc:
        out.put((rank, f"raised: {exc}"))
    except Exception as exc:  # noqa: BLE001  (the surviving ranks: a timed-out or broken collective)
        out.put((rank, f"collective failed: {type(exc).__name__}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def test_a_rank_that_raises_before_the_handoff_does_not_hang_the_others():
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=90) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res[1].startswith("raised: injected failure")
    for r in (0, 2):
        assert res[r].startswith("collective failed"), res
