#!/usr/bin/env python3
"""Benchmark of the state-space operator hot path on B200.

Default workload ("prefill"): one whole forward pass of a 64-layer Mamba-2 language model (d_model 2560,
expand 2, 80 heads x 64, d_state 128, one B/C group, chunk 256, conv width 4, RMSNorm, vocabulary 50280 with a tied
head; random-init bf16 weights, fp32 residual stream and states) over batch 2 x 131072 uniform random token ids.
The sequence is split into contiguous shards over the ranks (strong scaling): per layer the last K-1 conv inputs
travel to the next rank and the state-space-dual scan hands its chunk state over with one all-gather
(`ssm_b200.seqpar`).  One "step" is one such forward; the metric is tokens per second (batch * seqlen / step time).
The operators run on this repository's CUDA library, the dense projections on cuBLAS.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Under ``torch.distributed.run`` there is one rank per GPU; the timed region is bracketed by a barrier and a device
synchronisation, the maximum over ranks is reported by rank 0 as ONE JSON line.  That line also carries, inside
``roofline``, CUDA-event timings of every other operator configuration of the hot path (prefill scan, Mamba-1 block,
state-space-dual scan, decode steps, element-wise chunk scan) measured in the same process on one GPU, each with its
fraction of the measured HBM copy bandwidth.  ``--impl reference`` times the CPU restatement of the upstream Python
operators (oracle/) on the host cores for the same metric and prints the same line with ``"impl": "reference"``.
``--workload`` selects one of the operator configurations as the headline of the line instead.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

BLOCK_CFG = dict(batch=8, seqlen=4096, d_model=768, d_inner=1536, d_state=16, d_conv=4, dt_rank=48)
LM_CFG = dict(d_model=2560, n_layer=64, vocab_size=50280, batch=2, seqlen=131072, d_state=128, headdim=64, chunk_size=256, d_conv=4)


# --------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------
def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", 1440.6)), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def time_cuda(fn, steps, warmup=3):
    """Mean milliseconds per call over `steps` back-to-back calls, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def graph_time(fn, reps=4, iters=10):
    """Milliseconds per call of `fn` when `reps` calls are captured into one CUDA graph and replayed: device time only, none of
    the host-side launch work that an eager loop over a short kernel would measure."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(2):
            fn(i)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(reps):
            fn(i)
    return time_cuda(graph.replay, iters, 2) / reps


class CallTimer:
    """CUDA-event timing and counting of selected host entry points inside a timed region (on the launching stream)."""

    def __init__(self):
        self.events: dict[str, list] = {}
        self.calls: dict[str, int] = {}
        self.enabled = False
        self._undo = []

    def wrap(self, owner, name, tag, timed=True):
        inner = getattr(owner, name)
        timer = self

        def wrapped(*a, **k):
            if not timer.enabled:
                return inner(*a, **k)
            key = tag(*a, **k) if callable(tag) else tag
            timer.calls[key] = timer.calls.get(key, 0) + 1
            if not timed:
                return inner(*a, **k)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = inner(*a, **k)
            e1.record()
            timer.events.setdefault(key, []).append((e0, e1))
            return out

        setattr(owner, name, wrapped)
        self._undo.append((owner, name, inner))

    def restore(self):
        for owner, name, inner in self._undo:
            setattr(owner, name, inner)
        self._undo = []

    def mean_ms(self, tag):
        ev = self.events.get(tag, [])
        return sum(a.elapsed_time(b) for a, b in ev) / len(ev) if ev else None

    def total_ms(self, tag):
        return sum(a.elapsed_time(b) for a, b in self.events.get(tag, []))


# kernels launched by one call of a C-ABI entry point (ssm_ssd_fwd: by phase)
KERNELS_PER_CALL = {"ssm_selective_scan_fwd": 1, "ssm_selective_scan_bwd": 1, "ssm_selective_state_step": 1, "ssm_dw_causal_conv_fwd": 1,
                    "ssm_dw_causal_conv_bwd": 1, "ssm_dw_causal_conv_update": 1, "ssm_fused_add_norm_fwd": 1, "ssm_fused_add_norm_bwd": 2,
                    "ssm_chunk_scan_fwd": 3, "ssm_chunk_scan_bwd": 1, "ssm_ssd_fwd": 3, "ssm_ssd_fold_shards": 1, "ssm_mamba1_decode": 1}


def count_launches(timer: CallTimer) -> int:
    return sum(KERNELS_PER_CALL.get(k, 1) * v for k, v in timer.calls.items() if k.startswith("ssm_"))


def wrap_abi_calls(timer: CallTimer):
    """Count every C-ABI call made through `ssm_b200.ops` (each launches the kernels listed in KERNELS_PER_CALL)."""
    from ssm_b200 import ops

    inner = ops._call

    def counted(fn, args):
        if timer.enabled:
            name = getattr(fn, "__name__", None) or getattr(fn, "name", "ssm_call")
            timer.calls[name] = timer.calls.get(name, 0) + 1
        return inner(fn, args)

    ops._call = counted
    timer._undo.append((ops, "_call", inner))


# --------------------------------------------------------------------------------------
# default workload: sequence-sharded prefill of the 64-layer Mamba-2 model
# --------------------------------------------------------------------------------------
def build_lm(cfg, device, dtype, ops=None, seed=1234):
    from ssm_b200.lm import MambaConfig, MambaLMHeadModel

    if device != "cpu":
        torch.cuda.manual_seed(seed)  # the same weights on every rank
    torch.manual_seed(seed)
    mc = MambaConfig(d_model=cfg["d_model"], n_layer=cfg["n_layer"], vocab_size=cfg["vocab_size"],
                     ssm_cfg=dict(layer="Mamba2", d_state=cfg["d_state"], headdim=cfg["headdim"], chunk_size=cfg["chunk_size"], d_conv=cfg["d_conv"]))
    model = MambaLMHeadModel(mc, device=device, dtype=dtype, ops=ops)
    return model.eval()


def ssd_bytes(nb, nl, nh, hp=64, n=128, io=2):
    """Algorithmic HBM bytes of one state-space-dual scan: X, z in, Y out, dt, B, C in, final state out."""
    return 3 * nb * nl * nh * hp * io + nb * nl * nh * io + 2 * nb * nl * n * io + nb * nh * hp * n * 4


def ssd_flops(nb, nl, nh, hp=64, n=128, q=256):
    chunks = (nl + q - 1) // q
    return nb * chunks * nh * (2 * q * q * hp + 4 * q * n * hp) + nb * chunks * 2 * q * q * n


def run_prefill(args):
    import torch.distributed as dist

    from ssm_b200 import _lib, ops

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    under_launcher = "RANK" in os.environ
    if under_launcher:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    cfg = dict(LM_CFG)
    if args.layers:
        cfg["n_layer"] = args.layers
    if args.seqlen:
        cfg["seqlen"] = args.seqlen
    B, Ltot = cfg["batch"], cfg["seqlen"]
    Lq = Ltot // world
    nh = 2 * cfg["d_model"] // cfg["headdim"]
    model = build_lm(cfg, dev, torch.bfloat16)
    gi = torch.Generator().manual_seed(99)
    ids_all = torch.randint(0, cfg["vocab_size"], (B, Ltot), generator=gi)
    ids_host = ids_all[:, rank * Lq:(rank + 1) * Lq].contiguous().pin_memory()
    ids_dev = ids_host.to(dev)
    if rank == 0:
        print(f"[prefill] {cfg['n_layer']} layers ready: shard length {Lq}", file=sys.stderr, flush=True)

    timer = CallTimer()
    timer.wrap(ops._SsdWorkspace, "run", lambda self, phase, *a, **k: f"ssd_phase{phase}")
    wrap_abi_calls(timer)

    @torch.no_grad()
    def forward(ids):
        return model(ids, num_last_tokens=1, sharded=world > 1).logits[:, 0]  # logits of the shard's last token

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    steps = args.steps or 5
    tw = time.perf_counter()
    for i in range(args.warmup):
        forward(ids_dev)
        torch.cuda.synchronize()
        if rank == 0:
            print(f"[prefill] warm-up {i}: {time.perf_counter() - tw:.2f} s since start", file=sys.stderr, flush=True)

    def timed(fn):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    sampler = ClockSampler(local).start() if rank == 0 else None
    timer.enabled = True
    ms = timed(lambda: forward(ids_dev))
    timer.enabled = False
    out_host = torch.empty(B, model.lm_head.weight.shape[0], dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        logits = forward(ids_host.to(dev, non_blocking=True))
        out_host.copy_(logits, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    ms_e2e = timed(e2e_step)
    clocks = sampler.stop() if rank == 0 else None
    ops.ssd_check_status()

    # the state-space-dual operator on its own at this rank count (the part of a layer that carries the hand-off)
    sp_ms, sp_clocks = bench_ssd_sharded(rank, world, local, dev)
    extras = {}
    if rank == 0 and world == 1 and not args.no_extras:
        extras = operator_table(args)

    if rank == 0:
        tokens = B * Ltot
        peak, tpeak, kind = measured_peaks()
        calls = sum(timer.calls.get(f"ssd_phase{p}", 0) for p in (0, 1, 2))
        layer_calls = max(1, timer.calls.get("ssd_phase0", 0) + timer.calls.get("ssd_phase2", 0))
        ssd_ms = sum(timer.total_ms(f"ssd_phase{p}") for p in (0, 1, 2)) / layer_calls
        by = ssd_bytes(B, Lq, nh)
        fl = ssd_flops(B, Lq, nh)
        achieved = by / (ssd_ms * 1e-3) / 1e9
        roof = {"kernel": "ssm_ssd_fwd (cumsum + state + scan kernels of one state-space-dual scan, per layer and rank)", "bound": "hbm",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": kind,
                # dram__bytes_read.sum + dram__bytes_write.sum of the three kernels captured with ncu at batch 2 x 8192 x 48 heads
                # (profiles/ssd_kernels_ncu_batch2.md), scaled by the token-head count of this launch
                "traffic": TRAFFIC_PER_TOKEN_HEAD * B * Lq * nh, "bytes_per_launch": by, "ms_per_launch": ssd_ms,
                "tensor_tflops": fl / (ssd_ms * 1e-3) / 1e12, "tensor_frac_of_sustained_bf16": fl / (ssd_ms * 1e-3) / 1e12 / tpeak,
                "ssd_state_phase_ms": timer.mean_ms("ssd_phase1"), "ssd_scan_phase_ms": timer.mean_ms("ssd_phase2"),
                "ssd_share_of_step": ssd_ms * cfg["n_layer"] / ms, "sp_ssd_ms": sp_ms, "sp_ssd_clock_samples": sp_clocks}
        roof.update(extras)
        line = {
            "metric": "tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 weights / activations, fp32 residual stream and states", "data": "synthetic (seeded uniform token ids, random-init weights)",
            "config": {"workload": f"mamba2 prefill: {cfg['n_layer']} layers, d_model {cfg['d_model']}, {nh} heads x {cfg['headdim']}, d_state {cfg['d_state']}, "
                                   f"chunk {cfg['chunk_size']}, conv {cfg['d_conv']}, vocab {cfg['vocab_size']}; batch {B}, seqlen {Ltot} in {world} contiguous shards",
                       "parallelism": f"sp{world}: per layer a {cfg['d_conv'] - 1}-token conv halo to the next rank and an all-gather of the chunk state (5.2 MB / rank)",
                       "l2": "per-layer activations (GBs) exceed the 126 MB L2"},
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": ids_host.numel() * 8,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": count_launches(timer),
            "roofline": roof, "clocks": clocks,
        }
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline(budget_s=args.cpu_seconds)
        print(json.dumps(line))
    if under_launcher:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes per (token, head) of the three state-space-dual kernels, from the ncu capture named in `roofline.traffic`
TRAFFIC_PER_TOKEN_HEAD = 572.3e6 / (2 * 8192 * 48)


def bench_ssd_sharded(rank, world, local, dev, total_len=131072, steps=0):
    """The sequence-sharded state-space-dual scan alone: batch 2, 80 heads x 64, d_state 128, the shard of a `total_len`-token
    sequence this rank holds; strong scaling, max-over-ranks device time per call (ms) and the clock samples seen."""
    import torch.distributed as dist

    from ssm_b200 import seqpar

    B, H, P, N = 2, 80, 64, 128
    Lq = total_len // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    bf = torch.bfloat16
    X = torch.randn(B, Lq, H, P, generator=g, device=dev, dtype=bf)
    z = torch.randn(B, Lq, H, P, generator=g, device=dev, dtype=bf)
    dt = (torch.randn(B, Lq, H, generator=g, device=dev) - 3).to(bf)
    Bm = (torch.randn(B, Lq, 1, N, generator=g, device=dev) / N ** 0.5).to(bf)
    Cm = (torch.randn(B, Lq, 1, N, generator=g, device=dev) / N ** 0.5).to(bf)
    g0 = torch.Generator().manual_seed(7)
    A = (-torch.exp(torch.rand(H, generator=g0) * 2.7726)).to(dev)
    D = torch.randn(H, generator=g0).to(dev)

    @torch.no_grad()
    def step():
        return seqpar.ssd_scan_sharded(X, dt, A, Bm, Cm, 256, D=D, z=z, dt_softplus=True)

    steps = steps or max(40, 40 * world)  # long enough for the clock sampler at every rank count
    for _ in range(5):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local).start() if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    return float(t[0]), (clocks or {}).get("samples")


# --------------------------------------------------------------------------------------
# operator configurations measured beside the default workload (one GPU)
# --------------------------------------------------------------------------------------
def make_block_weights(cfg, device, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    dm, di, n, k, r = cfg["d_model"], cfg["d_inner"], cfg["d_state"], cfg["d_conv"], cfg["dt_rank"]

    def lin(o, i):
        return (torch.randn(o, i, generator=g) / i ** 0.5).to(dtype)

    w = dict(
        in_x=lin(di, dm), in_z=lin(di, dm), conv_w=(torch.rand(di, k, generator=g) - 0.5).to(dtype), conv_b=torch.zeros(di, dtype=dtype),
        x_proj=lin(r + 2 * n, di), dt_proj=lin(di, r),
        dt_bias=(torch.rand(di, generator=g) * 2 - 4).float(),  # softplus^-1 of a small positive step
        A=(-torch.exp(torch.randn(di, n, generator=g) * 0.5)).float(), D=torch.randn(di, generator=g).float(),
        out_proj=lin(dm, di), norm_w=torch.ones(dm, dtype=dtype),
    )
    return {k_: v.to(device).requires_grad_(True) for k_, v in w.items()}


def scan_bytes(b, d, l, n, io, bwd):
    """Algorithmic HBM bytes of one selective-scan launch: every input read once, every output written once (B / C are
    shared by all channels of a batch row)."""
    if not bwd:  # u, delta, z in; out; B, C; A, D, bias; last state
        return 4 * b * d * l * io + 2 * b * n * l * io + d * n * 4 + 2 * d * 4
    # u, delta, z, dout in; du, ddelta, dz out; B, C in; dB, dC out (fp32); dA, dD, dbias
    return 7 * b * d * l * io + 2 * b * n * l * io + 2 * b * n * l * 4 + 2 * d * n * 4 + 4 * d * 4


def bench_prefill_scan(iters=100):
    """selective_scan forward at batch 1, d_inner 512, seqlen 2048, d_state 16, fp32 (gate, skip, softplus, last state);
    the input sets rotate over more than the L2 holds."""
    from ssm_b200 import ops

    dev = torch.device("cuda")
    torch.manual_seed(0)
    nb, nd, nl, nn = 1, 512, 2048, 16
    nsets = 10
    sets = [dict(u=torch.randn(nb, nd, nl, device=dev), delta=torch.nn.functional.softplus(torch.randn(nb, nd, nl, device=dev) - 2),
                 B=torch.randn(nb, 1, nn, nl, device=dev), C=torch.randn(nb, 1, nn, nl, device=dev), z=torch.randn(nb, nd, nl, device=dev))
            for _ in range(nsets)]
    A, D = -torch.exp(torch.randn(nd, nn, device=dev) * 0.5), torch.randn(nd, device=dev)

    @torch.no_grad()
    def step(i):
        s = sets[i % nsets]
        return ops.selective_scan(s["u"], s["delta"], A, s["B"], s["C"], D=D, z=s["z"], softplus=True, return_last_state=True)

    ms = graph_time(step, reps=nsets, iters=max(2, iters // nsets))  # device time: the kernel is shorter than its eager host call
    by = 3 * nb * nd * nl * 4 + 2 * nb * nn * nl * 4 + nd * nn * 4 + nd * 4 + nb * nd * nl * 4 + nb * nd * nn * 4
    return {"ms": ms, "bytes": by}


def bench_mamba1_block(batch=8, steps=10, warmup=3, timer=None):
    """Forward + backward of a Mamba-1 mixer block (d_model 768, d_inner 1536, d_state 16, conv 4, dt_rank 48, bf16,
    fused add + RMSNorm) at seqlen 4096; CUDA events around the scan, conv and norm operator calls."""
    from ssm_b200 import ops
    from ssm_b200.mixer import mamba1_block_forward

    dev = torch.device("cuda")
    cfg = dict(BLOCK_CFG, batch=batch)
    B, Lq, dm = cfg["batch"], cfg["seqlen"], cfg["d_model"]
    w = make_block_weights(cfg, dev, torch.bfloat16, seed=0)
    own = timer is None
    timer = timer or CallTimer()
    timer.wrap(ops, "_scan_forward", "scan_fwd")
    timer.wrap(ops, "_scan_backward", "scan_bwd")
    timer.wrap(ops._ConvFn, "forward", "conv_fwd")
    timer.wrap(ops._ConvFn, "backward", "conv_bwd")
    timer.wrap(ops._NormFn, "forward", "norm_fwd")
    timer.wrap(ops._NormFn, "backward", "norm_bwd")
    g = torch.Generator().manual_seed(1234)
    xs = [torch.randn(B, Lq, dm, generator=g).to(torch.bfloat16).to(dev) for _ in range(2)]
    rs = [torch.randn(B, Lq, dm, generator=g).to(dev) for _ in range(2)]

    def step(i):
        for p in w.values():
            p.grad = None
        y, new_r = mamba1_block_forward(ops, w, cfg, xs[i % 2], rs[i % 2])
        loss = y.float().square().mean() + new_r.square().mean() * 1e-3
        loss.backward()
        return loss

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    timer.enabled = True
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    timer.enabled = False
    res = {"step_ms": e0.elapsed_time(e1) / steps, "tokens": B * Lq}
    for tag in ("scan_fwd", "scan_bwd", "conv_fwd", "conv_bwd", "norm_fwd", "norm_bwd"):
        res[tag + "_ms"] = timer.mean_ms(tag)
    d, n = cfg["d_inner"], cfg["d_state"]
    res["scan_fwd_bytes"] = scan_bytes(B, d, Lq, n, 2, False)
    res["scan_bwd_bytes"] = scan_bytes(B, d, Lq, n, 2, True)
    res["conv_fwd_bytes"] = 2 * B * d * Lq * 2
    res["conv_bwd_bytes"] = 3 * B * d * Lq * 2
    res["norm_fwd_bytes"] = B * Lq * dm * (2 + 4 + 2 + 4)   # x, fp32 residual in; y, fp32 residual out
    res["norm_bwd_bytes"] = B * Lq * dm * (2 + 4 + 2 + 4 + 2 + 4)  # x, residual, dy, d(residual out) in; dx, dresidual out
    if own:
        timer.restore()
    return res


def bench_conv_norm():
    """The depthwise causal conv (channel-major (8, 1536, 4096) bf16 rows, width 4, SiLU) and the fused add + RMSNorm ((32768, 768) bf16 with
    an fp32 residual stream in and out), forward and backward, as CUDA-graph replays over two alternating input sets."""
    from ssm_b200 import ops

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(5)
    kw = dict(generator=g, device=dev)
    bf = torch.bfloat16
    B, D, Lq, dm = 8, 1536, 4096, 768
    xs = [torch.randn(D, B, Lq, **kw).to(bf).permute(1, 0, 2).requires_grad_(True) for _ in range(2)]
    gys = [torch.randn(D, B, Lq, **kw).to(bf).permute(1, 0, 2) for _ in range(2)]
    cw, cb = (torch.rand(D, 4, **kw) - 0.5).requires_grad_(True), torch.zeros(D, device=dev, requires_grad=True)
    nx = [torch.randn(B, Lq, dm, **kw).to(bf).requires_grad_(True) for _ in range(2)]
    nr = [torch.randn(B, Lq, dm, **kw).requires_grad_(True) for _ in range(2)]
    ngy = [torch.randn(B, Lq, dm, **kw).to(bf) for _ in range(2)]
    ngr = [torch.randn(B, Lq, dm, **kw) for _ in range(2)]
    nw = torch.ones(dm, device=dev, dtype=bf, requires_grad=True)

    def conv_fwd(i):
        with torch.no_grad():
            return ops.dw_causal_conv(xs[i % 2], cw, cb, "silu")

    def conv_both(i):
        y = ops.dw_causal_conv(xs[i % 2], cw, cb, "silu")
        return torch.autograd.grad(y, (xs[i % 2], cw, cb), gys[i % 2])

    def norm_fwd(i):
        with torch.no_grad():
            return ops.fused_layer_norm(nx[i % 2], nw, None, residual=nr[i % 2], is_rms=True, prenorm=True, return_residual=True)

    def norm_both(i):
        y, ro = ops.fused_layer_norm(nx[i % 2], nw, None, residual=nr[i % 2], is_rms=True, prenorm=True, return_residual=True)
        return torch.autograd.grad((y, ro), (nx[i % 2], nr[i % 2], nw), (ngy[i % 2], ngr[i % 2]))

    cf, cfb, nf, nfb = graph_time(conv_fwd), graph_time(conv_both), graph_time(norm_fwd), graph_time(norm_both)
    el_c, el_n = B * D * Lq, B * Lq * dm
    return {"conv_fwd_ms": cf, "conv_bwd_ms": cfb - cf, "norm_fwd_ms": nf, "norm_bwd_ms": nfb - nf,
            "conv_fwd_bytes": 2 * el_c * 2, "conv_bwd_bytes": 3 * el_c * 2,
            "norm_fwd_bytes": el_n * (2 + 4 + 2 + 4),            # x, fp32 residual in; y, fp32 residual stream out
            "norm_bwd_bytes": el_n * (2 + 4 + 2 + 4 + 2 + 4)}    # x, residual, dy, d(residual stream) in; dx, dresidual out


def bench_mamba2_layer_ops():
    """The bandwidth kernels of one Mamba-2 layer on the shard one of eight ranks holds (32768 tokens, d_model 2560, d_inner 5120):
    channels-last conv + SiLU over 5120 and over 128 channels, RMSNorm over 5120 columns, fused add + RMSNorm over 2560 columns with the
    fp32 residual stream in and out; forward, CUDA-graph replays over two alternating input sets."""
    from ssm_b200 import ops

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(6)
    kw = dict(generator=g, device=dev)
    bf = torch.bfloat16
    B, Lq, dm, di, n = 2, 16384, 2560, 5120, 128
    cx = [torch.randn(B, Lq, di, **kw).to(bf) for _ in range(2)]
    cb = [torch.randn(B, Lq, n, **kw).to(bf) for _ in range(2)]
    wx, wb = torch.rand(di, 4, **kw) - 0.5, torch.rand(n, 4, **kw) - 0.5
    nx = [torch.randn(B, Lq, dm, **kw).to(bf) for _ in range(2)]
    nr = [torch.randn(B, Lq, dm, **kw) for _ in range(2)]
    w_dm, w_di = torch.ones(dm, device=dev, dtype=bf), torch.ones(di, device=dev, dtype=bf)

    @torch.no_grad()
    def conv_x(i):
        return ops.dw_causal_conv(cx[i % 2], wx, None, "silu")

    @torch.no_grad()
    def conv_b(i):
        return ops.dw_causal_conv(cb[i % 2], wb, None, "silu")

    @torch.no_grad()
    def norm_wide(i):
        return ops.fused_layer_norm(cx[i % 2], w_di, None, is_rms=True)

    @torch.no_grad()
    def add_norm(i):
        return ops.fused_layer_norm(nx[i % 2], w_dm, None, residual=nr[i % 2], is_rms=True, prenorm=True, return_residual=True)

    # backward of the wide conv (what training a Mamba-2 layer adds): forward + backward minus forward
    cxg = [t.clone().requires_grad_(True) for t in cx]
    wxg = wx.clone().requires_grad_(True)
    gyc = [torch.randn(B, Lq, di, **kw).to(bf) for _ in range(2)]

    def conv_x_both(i):
        y = ops.dw_causal_conv(cxg[i % 2], wxg, None, "silu")
        return torch.autograd.grad(y, (cxg[i % 2], wxg), gyc[i % 2])

    rows = B * Lq
    t_conv = graph_time(conv_x)
    return {"conv_cl_5120_ms": t_conv, "conv_cl_5120_bytes": 2 * rows * di * 2,
            "conv_cl_5120_bwd_ms": graph_time(conv_x_both) - t_conv, "conv_cl_5120_bwd_bytes": 3 * rows * di * 2,
            "conv_cl_128_ms": graph_time(conv_b), "conv_cl_128_bytes": 2 * rows * n * 2,
            "norm_5120_ms": graph_time(norm_wide), "norm_5120_bytes": 2 * rows * di * 2,
            "add_norm_2560_ms": graph_time(add_norm), "add_norm_2560_bytes": rows * dm * (2 + 4 + 2 + 4)}


def bench_ssd(batch=8, steps=20):
    """State-space-dual scan forward: seqlen 8192, 48 heads x 64, d_state 128, one group, chunk 256, bf16."""
    from ssm_b200 import ops

    dev = torch.device("cuda")
    B, Lq, H, P, N = batch, 8192, 48, 64, 128
    g = torch.Generator(device=dev).manual_seed(0)
    kw = dict(generator=g, device=dev)
    bf = torch.bfloat16
    t = dict(X=torch.randn(B, Lq, H, P, **kw).to(bf), dt=(torch.randn(B, Lq, H, **kw) - 3).to(bf), Bm=(torch.randn(B, Lq, 1, N, **kw) / N ** 0.5).to(bf),
             Cm=(torch.randn(B, Lq, 1, N, **kw) / N ** 0.5).to(bf), z=torch.randn(B, Lq, H, P, **kw).to(bf))
    A = -torch.exp(torch.rand(H, **kw) * 2.7726)
    D = torch.randn(H, **kw)

    @torch.no_grad()
    def step():
        return ops.ssd_scan(t["X"], t["dt"], A, t["Bm"], t["Cm"], 256, D=D, z=t["z"], dt_softplus=True, return_final_states=True)

    ms = time_cuda(step, steps, 3)
    # backward in the dual form (four more runs of the tensor-core kernels on transformed operands): gradients of every
    # input for a given output gradient, forward excluded from the timed region
    lv = {k: v.clone().requires_grad_(True) for k, v in t.items()}
    Ag, Dg = A.clone().requires_grad_(True), D.clone().requires_grad_(True)
    gy = torch.randn(B, Lq, H, P, **kw).to(bf)
    Y = ops.ssd_scan(lv["X"], lv["dt"], Ag, lv["Bm"], lv["Cm"], 256, D=Dg, z=lv["z"], dt_softplus=True)
    leaves = [lv["X"], lv["dt"], Ag, lv["Bm"], lv["Cm"], Dg, lv["z"]]
    bwd_ms = time_cuda(lambda: torch.autograd.grad(Y, leaves, gy, retain_graph=True), max(3, steps // 4), 2)
    return {"ms": ms, "bwd_ms": bwd_ms, "bytes": ssd_bytes(B, Lq, H), "flops": ssd_flops(B, Lq, H), "tokens": B * Lq}


def bench_decode(steps=1000):
    """Single-token steps at batch 256: the Mamba-1 layer (d_model 2560, d_inner 5120, d_state 16, conv 4, dt_rank 160; fp32 states,
    bf16 activations) eagerly and as CUDA-graph replays, its two state kernels alone over rotating state buffers (so the 84 MB state
    cannot stay in the L2), and the Mamba-2 state step (80 heads x 64, d_state 128)."""
    from ssm_b200 import ops
    from ssm_b200.mixer import mamba1_mixer_step

    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(0)
    B, dm, di, n, k, r = 256, 2560, 5120, 16, 4, 160
    bf = torch.bfloat16
    lin = lambda o, i: (torch.randn(o, i, generator=g) / i ** 0.5).to(bf).to(dev)  # noqa: E731
    w = dict(in_x=lin(di, dm), in_z=lin(di, dm), x_proj=lin(r + 2 * n, di), dt_proj=lin(di, r), out_proj=lin(dm, di),
             conv_w=(torch.rand(di, k, generator=g) - 0.5).to(dev), conv_b=None, A=(-torch.exp(torch.randn(di, n, generator=g) * 0.5)).to(dev),
             D=torch.randn(di, generator=g).to(dev), dt_bias=(torch.rand(di, generator=g) * 2 - 4).to(dev))
    cfg = dict(d_state=n, dt_rank=r)
    nbuf = 3  # 3 x (84 + 21) MB of state: more than the 126 MB L2
    ssm = [(torch.randn(B, di, n, generator=g) * 0.1).to(dev) for _ in range(nbuf)]
    conv = [(torch.randn(B, di, k, generator=g) * 0.1).to(dev) for _ in range(nbuf)]
    tok = torch.randn(B, dm, generator=g).to(bf).to(dev)
    it = [0]

    @torch.no_grad()
    def layer_step():
        i = it[0] % nbuf
        it[0] += 1
        return mamba1_mixer_step(ops, w, cfg, tok, conv[i], ssm[i])

    xs, ds, zs = (torch.randn(B, di, generator=g).to(bf).to(dev) for _ in range(3))
    Bf, Cf = torch.randn(B, 1, n, generator=g).to(bf).to(dev), torch.randn(B, 1, n, generator=g).to(bf).to(dev)

    @torch.no_grad()
    def state_kernels():
        i = it[0] % nbuf
        it[0] += 1
        u = ops.dw_causal_conv_update(conv[i], xs, w["conv_w"], None, "silu")
        return ops.selective_state_step(ssm[i], u, ds, w["A"], Bf, Cf, D=w["D"], z=zs, dt_bias=w["dt_bias"], softplus=True)

    H2, P2, N2 = 80, 64, 128
    st2 = [(torch.randn(B, H2, P2, N2, generator=g) * 0.1).to(dev) for _ in range(2)]
    x2, z2 = torch.randn(B, H2, P2, generator=g).to(bf).to(dev), torch.randn(B, H2, P2, generator=g).to(bf).to(dev)
    dt2, A2 = torch.randn(B, H2, generator=g).to(bf).to(dev), (-torch.exp(torch.rand(H2, generator=g))).to(dev)
    B2, C2 = torch.randn(B, 1, N2, generator=g).to(bf).to(dev), torch.randn(B, 1, N2, generator=g).to(bf).to(dev)
    D2 = torch.randn(H2, generator=g).to(dev)

    @torch.no_grad()
    def m2_step():
        it[0] += 1
        return ops.selective_state_step_heads(st2[it[0] % 2], x2, dt2, A2, B2, C2, D=D2, z=z2, softplus=True)

    def state_kernels_i(i):
        it[0] = i
        state_kernels()

    def m2_step_i(i):
        it[0] = i
        m2_step()

    res = {"layer_eager_us": time_cuda(layer_step, steps, 20) * 1e3, "state_kernels_us": graph_time(state_kernels_i, reps=2 * nbuf, iters=50) * 1e3,
           "mamba2_step_us": graph_time(m2_step_i, reps=4, iters=20) * 1e3}
    # CUDA-graph replay of the whole layer step (one fixed pair of state buffers, as a decoder has)
    try:
        it[0] = 0
        gph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                it[0] = 0
                layer_step()
        torch.cuda.current_stream().wait_stream(side)
        it[0] = 0
        with torch.cuda.graph(gph):
            layer_step()
        res["layer_graph_us"] = time_cuda(gph.replay, steps, 20) * 1e3
    except Exception as exc:  # noqa: BLE001
        res["layer_graph_us"] = None
        res["layer_graph_error"] = str(exc)[:200]
    # state r+w, conv window r+w, x / delta / z in, u / y out, B, C, A
    res["state_kernels_bytes"] = 2 * B * di * n * 4 + 2 * B * di * k * 4 + 5 * B * di * 2 + 2 * B * n * 2 + di * n * 4
    res["mamba2_step_bytes"] = 2 * B * H2 * P2 * N2 * 4 + 3 * B * H2 * P2 * 2
    return res


def bench_chunk_scan(steps=20):
    """Element-wise chunked recurrence (upstream's `ssd_chunk_scan`), forward and backward, at the two shapes of upstream's
    operator benchmark (benchmarks/ops_bench.py:100-117): batch 8, seqlen 2048, 16 heads x 64, chunk 128 and
    batch 4, seqlen 4096, 32 heads x 64, chunk 256; bf16, per-token B / C, gate, skip."""
    from ssm_b200 import ops

    dev = torch.device("cuda")
    out = {}
    for name, (B, Lq, H, P, chunk) in dict(l2k_h16_c128=(8, 2048, 16, 64, 128), l4k_h32_c256=(4, 4096, 32, 64, 256)).items():
        g = torch.Generator(device=dev).manual_seed(3)
        kw = dict(generator=g, device=dev)
        bf = torch.bfloat16
        sets = []
        for _ in range(3):  # 3 x ~170 MB of operands: more than the L2
            sets.append(dict(X=torch.randn(B, Lq, H, P, **kw).to(bf).requires_grad_(True), dt=(torch.rand(B, Lq, H, **kw) * 0.1).to(bf),
                             Bm=torch.randn(B, Lq, H, P, **kw).to(bf), Cm=torch.randn(B, Lq, H, P, **kw).to(bf), z=torch.randn(B, Lq, H, P, **kw).to(bf),
                             gY=torch.randn(B, Lq, H, P, **kw).to(bf)))
        A, D = -torch.exp(torch.randn(H, P, **kw) * 0.5), torch.randn(H, **kw)
        for st in sets:
            for k_ in ("Bm", "Cm", "z"):
                st[k_].requires_grad_(True)

        def fwd(i):
            s = sets[i % 3]
            with torch.no_grad():
                return ops.ssd_chunk_scan(s["X"], s["dt"], A, s["Bm"], s["Cm"], chunk, D=D, z=s["z"])

        def fwd_bwd(i):
            s = sets[i % 3]
            Y = ops.ssd_chunk_scan(s["X"], s["dt"], A, s["Bm"], s["Cm"], chunk, D=D, z=s["z"])
            return torch.autograd.grad(Y, (s["X"], s["Bm"], s["Cm"], s["z"]), s["gY"])

        f = graph_time(fwd, reps=3, iters=max(2, steps // 3))
        fb = graph_time(fwd_bwd, reps=3, iters=max(2, steps // 3))
        el = B * Lq * H * P
        out[name] = {"fwd_ms": f, "bwd_ms": fb - f, "fwd_bytes": 5 * el * 2 + B * Lq * H * 2, "bwd_bytes": 6 * el * 2 + B * Lq * H * 2 + B * Lq * H * 4}
    return out


def operator_table(args):
    """Flat scalar keys for the `roofline` object: one CUDA-event timing per operator configuration, with its fraction of the
    measured HBM copy bandwidth (algorithmic bytes / time / peak)."""
    peak, tpeak, _ = measured_peaks()
    frac = lambda by, ms: by / (ms * 1e-3) / 1e9 / peak  # noqa: E731
    t = {}
    c1 = bench_prefill_scan()
    t["c1_scan_fwd_us"], t["c1_scan_fwd_frac"] = c1["ms"] * 1e3, frac(c1["bytes"], c1["ms"])
    sampler = ClockSampler(torch.cuda.current_device()).start()
    c2 = bench_mamba1_block()
    t["c2_clocks"] = json.dumps(sampler.stop())
    t["c2_step_ms"] = c2["step_ms"]
    t["c2_tokens_per_s"] = c2["tokens"] / (c2["step_ms"] * 1e-3)
    for tag in ("scan_fwd", "scan_bwd"):
        t[f"c2_{tag}_ms"], t[f"c2_{tag}_frac"] = c2[tag + "_ms"], frac(c2[tag + "_bytes"], c2[tag + "_ms"])
    cn = bench_conv_norm()  # short kernels: device time from CUDA-graph replays, not from events around eager host calls
    for tag in ("conv_fwd", "conv_bwd", "norm_fwd", "norm_bwd"):
        t[f"c2_{tag}_ms"], t[f"c2_{tag}_frac"] = cn[tag + "_ms"], frac(cn[tag + "_bytes"], cn[tag + "_ms"])
    # the scan is bound by the special-function unit, not by HBM: one ex2 per (row, state, step) plus softplus / SiLU per (row, step)
    b, d, l, n = BLOCK_CFG["batch"], BLOCK_CFG["d_inner"], BLOCK_CFG["seqlen"], BLOCK_CFG["d_state"]
    xu_floor_ms = b * d * l * (n + 4) / (148 * 16 * 1.965e9) * 1e3
    t["c2_scan_fwd_xu_frac"] = xu_floor_ms / c2["scan_fwd_ms"]
    t["c2_scan_bwd_xu_frac"] = 2 * xu_floor_ms / c2["scan_bwd_ms"]
    c3 = bench_ssd()
    t["c3_ssd_ms"], t["c3_ssd_frac"], t["c3_ssd_tflops"] = c3["ms"], frac(c3["bytes"], c3["ms"]), c3["flops"] / (c3["ms"] * 1e-3) / 1e12
    t["c3_ssd_tokens_per_s"] = c3["tokens"] / (c3["ms"] * 1e-3)
    t["c3_ssd_bwd_ms"] = c3["bwd_ms"]
    c5 = bench_mamba2_layer_ops()  # the bandwidth kernels of one layer of the default workload at the 8-rank shard size
    for tag in ("conv_cl_5120", "conv_cl_5120_bwd", "conv_cl_128", "norm_5120", "add_norm_2560"):
        t[f"c5_{tag}_us"], t[f"c5_{tag}_frac"] = c5[tag + "_ms"] * 1e3, frac(c5[tag + "_bytes"], c5[tag + "_ms"])
    c4 = bench_decode()
    t["c4a_step_us"], t["c4a_step_frac"] = c4["state_kernels_us"], frac(c4["state_kernels_bytes"], c4["state_kernels_us"] * 1e-3)
    t["c4b_step_us"], t["c4b_step_frac"] = c4["mamba2_step_us"], frac(c4["mamba2_step_bytes"], c4["mamba2_step_us"] * 1e-3)
    t["c4_layer_us_eager"], t["c4_layer_us_graph"] = c4["layer_eager_us"], c4["layer_graph_us"]
    a4 = bench_chunk_scan()
    for name, r in a4.items():
        t[f"a4_{name}_fwd_ms"], t[f"a4_{name}_fwd_frac"] = r["fwd_ms"], frac(r["fwd_bytes"], r["fwd_ms"])
        t[f"a4_{name}_bwd_ms"], t[f"a4_{name}_bwd_frac"] = r["bwd_ms"], frac(r["bwd_bytes"], r["bwd_ms"])
    return t


# --------------------------------------------------------------------------------------
# CPU arm: the oracle (a restatement of the upstream Python operators) on the host cores
# --------------------------------------------------------------------------------------
def cpu_baseline(budget_s=15.0, steps=None, layers=4, seqlen=1024):
    """The same model forward on the CPU oracle, on a bounded sample: `layers` of the 64 layers, batch 1, `seqlen` tokens, fp32.
    tokens/s is scaled to the 64-layer model (time per layer x 64)."""
    from oracle import ssm_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = dict(LM_CFG, n_layer=layers)
    model = build_lm(cfg, "cpu", torch.float32, ops=orc)
    ids = torch.randint(0, cfg["vocab_size"], (1, seqlen), generator=torch.Generator().manual_seed(99))

    def step():
        with torch.no_grad():
            model(ids, num_last_tokens=1)

    step()  # warm-up
    n, t0 = 0, time.perf_counter()
    while True:
        step()
        n += 1
        el = time.perf_counter() - t0
        if (steps is not None and n >= steps) or (steps is None and (el > budget_s or n >= 20)):
            break
    per_layer = el / n / layers
    tok = seqlen / (per_layer * LM_CFG["n_layer"])
    return {"value": tok, "unit": "tokens/s", "cores": cores, "kind": "port", "seconds": el, "ms_per_pass": el / n * 1e3,
            "sample": f"{layers} of the 64 layers at batch 1, seqlen {seqlen} (fp32), {n} passes, scaled to 64 layers; upstream's CPU path is its "
                      "per-token Python loop, restated in oracle/ssm_oracle.py"}


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    steps = max(1, args.steps or 3)
    base = cpu_baseline(steps=steps)
    ms = base["ms_per_pass"]
    nh = 2 * LM_CFG["d_model"] // LM_CFG["headdim"]
    line = {
        "impl": "reference", "metric": "tokens_per_s", "value": base["value"], "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic (seeded)",
        "config": {"workload": f"mamba2 prefill: 64 layers, d_model {LM_CFG['d_model']}, {nh} heads x {LM_CFG['headdim']}, d_state {LM_CFG['d_state']} "
                               "(bounded sample: 4 layers, batch 1, seqlen 1024, scaled to 64 layers)", "parallelism": "host cores"},
        "cpu_baseline": base, "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# single-configuration headlines (--workload)
# --------------------------------------------------------------------------------------
def run_single(args):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, tpeak, kind = measured_peaks()
    steps = args.steps or 20
    sampler = ClockSampler(0).start()
    wl = args.workload
    roof, extra = {}, {}
    if wl == "mamba1_block":
        timer = CallTimer()
        wrap_abi_calls(timer)
        r = bench_mamba1_block(batch=args.batch or 8, steps=steps, warmup=args.warmup, timer=timer)
        ms, value, unit, metric, hib = r["step_ms"], r["tokens"] / (r["step_ms"] * 1e-3), "tokens/s", "tokens_per_s", True
        ach = r["scan_bwd_bytes"] / (r["scan_bwd_ms"] * 1e-3) / 1e9
        roof = {"kernel": "scan_bwd_kernel", "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_kind": kind,
                "traffic": 172.58e6 * (args.batch or 8) / 2, "bytes_per_launch": r["scan_bwd_bytes"], "ms_per_launch": r["scan_bwd_ms"]}
        for tag in ("scan_fwd", "conv_fwd", "conv_bwd", "norm_fwd", "norm_bwd"):
            roof[tag + "_ms"] = r[tag + "_ms"]
            roof[tag + "_frac"] = r[tag + "_bytes"] / (r[tag + "_ms"] * 1e-3) / 1e9 / peak
        extra["gpu_launches"] = count_launches(timer)
        timer.restore()
        work = f"mamba1_block fwd+bwd: batch {args.batch or 8}, seqlen 4096, d_model 768, d_inner 1536, d_state 16, d_conv 4, dt_rank 48, RMSNorm eps 1e-5"
    elif wl == "ssd":
        r = bench_ssd(batch=args.batch or 8, steps=steps)
        ms, value, unit, metric, hib = r["ms"], r["tokens"] / (r["ms"] * 1e-3), "tokens/s", "tokens_per_s", True
        ach = r["bytes"] / (ms * 1e-3) / 1e9
        roof = {"kernel": "ssm_ssd_fwd (cumsum + state + scan kernels)", "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                "peak_kind": kind, "traffic": TRAFFIC_PER_TOKEN_HEAD * r["tokens"] * 48, "bytes_per_launch": r["bytes"],
                "tensor_tflops": r["flops"] / (ms * 1e-3) / 1e12, "bwd_ms": r["bwd_ms"]}
        extra["gpu_launches"] = 3 * steps
        work = f"ssd chunk scan fwd: batch {args.batch or 8}, seqlen 8192, 48 heads x 64, d_state 128, ngroups 1, chunk 256"
    elif wl == "decode":
        r = bench_decode(steps=max(steps, 1000) if not args.steps else steps)
        val = r["layer_graph_us"] or r["layer_eager_us"]
        ms, value, unit, metric, hib = val * 1e-3, val, "us/step", "decode_step_us", False
        ach = r["state_kernels_bytes"] / (r["state_kernels_us"] * 1e-6) / 1e9
        roof = {"kernel": "conv_update_kernel + step_fwd_fast_kernel (Mamba-1 state 256 x 5120 x 16, conv window 256 x 5120 x 4)", "bound": "hbm",
                "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_kind": kind, "traffic": None,
                "us_per_launch_pair": r["state_kernels_us"], "layer_eager_us": r["layer_eager_us"], "layer_graph_us": r["layer_graph_us"],
                "mamba2_step_us": r["mamba2_step_us"], "mamba2_step_frac": r["mamba2_step_bytes"] / (r["mamba2_step_us"] * 1e-6) / 1e9 / peak}
        extra["gpu_launches"] = 2 * steps
        work = "decode: Mamba-1 layer step, batch 256, d_model 2560, d_inner 5120, d_state 16, conv 4, dt_rank 160; consecutive steps"
    elif wl == "scan_c1":
        r = bench_prefill_scan(iters=max(steps, 50))
        ms, value, unit, metric, hib = r["ms"], 2048 / (r["ms"] * 1e-3), "tokens/s", "tokens_per_s", True
        ach = r["bytes"] / (ms * 1e-3) / 1e9
        roof = {"kernel": "scan_fwd_tiles_kernel", "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_kind": kind,
                "traffic": None, "bytes_per_launch": r["bytes"]}
        extra["gpu_launches"] = max(steps, 50)
        work = "selective_scan fwd: batch 1, d_inner 512, seqlen 2048, d_state 16, fp32; 10 rotating input sets (171 MB) exceed the 126 MB L2"
    elif wl == "chunk_scan":
        r = bench_chunk_scan(steps=steps)["l4k_h32_c256"]
        ms, value, unit, metric, hib = r["fwd_ms"], 4 * 4096 / (r["fwd_ms"] * 1e-3), "tokens/s", "tokens_per_s", True
        ach = r["fwd_bytes"] / (ms * 1e-3) / 1e9
        roof = {"kernel": "chunk_local / chunk_carry / chunk_apply kernels", "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                "peak_kind": kind, "traffic": None, "bytes_per_launch": r["fwd_bytes"], "bwd_ms": r["bwd_ms"],
                "bwd_frac": r["bwd_bytes"] / (r["bwd_ms"] * 1e-3) / 1e9 / peak}
        extra["gpu_launches"] = 3 * steps
        work = "element-wise chunk scan fwd: batch 4, seqlen 4096, 32 heads x 64, chunk 256, bf16"
    else:
        raise SystemExit(f"unknown workload {wl}")
    clocks = sampler.stop()
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": 1, "steps": steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": hib, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 I/O, fp32 state" if wl != "scan_c1" else "fp32",
            "data": "synthetic (seeded)", "config": {"workload": work, "l2": "working set or rotating buffers exceed the 126 MB L2"},
            "roofline": roof, "clocks": clocks}
    line.update(extra)
    print(json.dumps(line))


def run_ssd_sp(args):
    """The sequence-sharded state-space-dual scan alone as the headline (strong scaling over the ranks)."""
    import torch.distributed as dist

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    under_launcher = "RANK" in os.environ
    if under_launcher:
        dist.init_process_group("nccl", device_id=dev)
    Ltot = args.seqlen or 131072
    ms, samples = bench_ssd_sharded(rank, world, local, dev, total_len=Ltot, steps=args.steps)
    if rank == 0:
        peak, _, kind = measured_peaks()
        by = ssd_bytes(2, Ltot // world, 80)
        print(json.dumps({
            "metric": "tokens_per_s", "value": 2 * Ltot / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps or max(40, 40 * world),
            "warmup": 5, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 operands, fp32 accumulate/state", "data": "synthetic (seeded)",
            "config": {"workload": f"sequence-sharded ssd scan: batch 2, seqlen {Ltot} in {world} contiguous shards, 80 heads x 64, d_state 128, chunk 256",
                       "parallelism": f"sp{world}: all-gather of (final state 5.2 MB, log-decay) per rank over NCCL, associative fold",
                       "l2": "per-GPU inputs exceed the 126 MB L2"},
            "gpu_launches": 4 * (args.steps or max(40, 40 * world)),
            "roofline": {"kernel": "ssm_ssd_fwd phases 1+2 per shard", "bound": "hbm", "achieved": by / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": by / (ms * 1e-3) / 1e9 / peak, "peak_kind": kind, "traffic": None},
            "clocks": {"samples": samples}}))
    if under_launcher:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="timed steps (default: 5 forward passes of the model; 20 for the operator workloads)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-operator table inside `roofline`")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--batch", type=int, default=0, help="override the batch of an operator workload (profiling on a smaller case)")
    ap.add_argument("--workload", default="prefill", choices=["prefill", "mamba1_block", "ssd", "decode", "scan_c1", "chunk_scan", "ssd_sp"])
    ap.add_argument("--layers", type=int, default=0, help="override the depth of the prefill workload")
    ap.add_argument("--seqlen", type=int, default=0, help="override the total sequence length of the prefill / ssd_sp workloads")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "ssd_sp":
        run_ssd_sp(args)
    else:
        run_single(args)


if __name__ == "__main__":
    main()
