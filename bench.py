#!/usr/bin/env python3
"""Benchmark of the state-space operator hot path on B200.

Default workload ("mamba1_block"): one forward + backward pass of a Mamba-1 mixer block at
batch 8, sequence 4096, d_model 768 (d_inner 1536, d_state 16, conv width 4, dt_rank 48, bf16
activations, fp32 scan state, fused residual-add + RMSNorm), i.e. conv -> x_proj -> dt_proj
-> selective scan -> out_proj -> add+norm and their gradients.  The five operators run on
this repository's CUDA library; the dense projections are cuBLAS matmuls.  Inputs are
seeded synthetic tensors with random-init weights.  One "step" is one such pass; the metric
is tokens per second (batch * seqlen / step time).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Under ``torch.distributed.run`` every rank runs the same per-GPU workload on its own batch
shard (weak scaling, no data-path collective); the timed region is bracketed by a barrier and
a device synchronisation and the maximum over ranks is reported by rank 0 as ONE JSON line.
``--impl reference`` times the CPU restatement of the upstream Python operators (oracle/)
on the host cores for the same metric and prints the same line with ``"impl": "reference"``.
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

CFG = dict(batch=8, seqlen=4096, d_model=768, d_inner=1536, d_state=16, d_conv=4, dt_rank=48)


# --------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------
def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
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
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# --------------------------------------------------------------------------------------
# the Mamba-1 block, written against an operator namespace (GPU library or CPU oracle)
# --------------------------------------------------------------------------------------
def make_weights(cfg, device, dtype, seed=0):
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


from ssm_b200.mixer import mamba1_block_forward as block_forward  # noqa: E402  (the block both arms run)


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
class KernelTimer:
    """CUDA-event timing of selected C-ABI calls inside the timed region (on the launching stream)."""

    def __init__(self):
        self.events: dict[str, list] = {}
        self.launches = 0
        self.enabled = False

    def wrap(self, module, name, tag, kernels):
        inner = getattr(module, name)
        timer = self

        def wrapped(*a, **k):
            if not timer.enabled:
                return inner(*a, **k)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = inner(*a, **k)
            e1.record()
            timer.events.setdefault(tag, []).append((e0, e1))
            timer.launches += kernels
            return out

        setattr(module, name, wrapped)

    def mean_ms(self, tag):
        ev = self.events.get(tag, [])
        return sum(a.elapsed_time(b) for a, b in ev) / len(ev) if ev else None


def scan_bytes(cfg, batch, bwd):
    """Algorithmic HBM bytes of one selective-scan launch at bf16 I/O: every input read once,
    every output written once (B/C are shared by all channels of a batch row)."""
    b, d, l, n = batch, cfg["d_inner"], cfg["seqlen"], cfg["d_state"]
    io = 2
    if not bwd:  # u, delta, z in; out
        return 4 * b * d * l * io + 2 * b * n * l * io + d * n * 4 + 2 * d * 4
    # u, delta, z, dout in; du, ddelta, dz out; B, C in; dB, dC out (fp32); dA, dD, dbias
    return 7 * b * d * l * io + 2 * b * n * l * io + 2 * b * n * l * 4 + 2 * d * n * 4 + 4 * d * 4


def run_gpu(args):
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    from ssm_b200 import _lib, ops

    _lib.load()
    cfg = dict(CFG)
    if args.batch:
        cfg["batch"] = args.batch
    B, Lq, dm = cfg["batch"], cfg["seqlen"], cfg["d_model"]
    w = make_weights(cfg, dev, torch.bfloat16, seed=0)
    timer = KernelTimer()
    timer.wrap(ops, "_scan_forward", "scan_fwd", 1)
    timer.wrap(ops, "_scan_backward", "scan_bwd", 1)
    # launches of the other operators are counted, not timed individually
    counted = {"conv_fwd": 1, "conv_bwd": 1, "norm_fwd": 1, "norm_bwd": 2}

    # host-resident inputs (pinned): a few distinct batches so that the copies are real
    g = torch.Generator().manual_seed(1234 + rank)
    nbuf = 2
    host_x = [torch.randn(B, Lq, dm, generator=g).to(torch.bfloat16).pin_memory() for _ in range(nbuf)]
    host_r = [torch.randn(B, Lq, dm, generator=g).pin_memory() for _ in range(nbuf)]
    dev_x = [t.to(dev) for t in host_x]
    dev_r = [t.to(dev) for t in host_r]
    h2d = host_x[0].numel() * 2 + host_r[0].numel() * 4
    loss_host = torch.empty(1, dtype=torch.float32).pin_memory()

    def step(x, r):
        for p in w.values():
            p.grad = None
        y, new_r = block_forward(ops, w, cfg, x, r)
        loss = y.float().square().mean() + new_r.square().mean() * 1e-3
        loss.backward()
        return loss

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ---------------------------------------------------------
    for i in range(args.warmup):
        step(dev_x[i % nbuf], dev_r[i % nbuf])
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    timer.enabled = True
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(dev_x[i % nbuf], dev_r[i % nbuf])
    e1.record()
    barrier()
    timer.enabled = False
    ms_dev = e0.elapsed_time(e1) / args.steps

    # ---- end to end: pinned host inputs -> device (prefetched on a copy stream) -> loss back ----
    copy_stream = torch.cuda.Stream()
    stage_x = [torch.empty_like(dev_x[0]) for _ in range(2)]
    stage_r = [torch.empty_like(dev_r[0]) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    done = [torch.cuda.Event() for _ in range(2)]

    def prefetch(i):
        s = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(done[s])
            stage_x[s].copy_(host_x[i % nbuf], non_blocking=True)
            stage_r[s].copy_(host_r[i % nbuf], non_blocking=True)
            ready[s].record(copy_stream)

    def e2e_loop(n):
        for s in range(2):
            done[s].record()
        prefetch(0)
        for i in range(n):
            s = i % 2
            if i + 1 < n:
                prefetch(i + 1)
            torch.cuda.current_stream().wait_event(ready[s])
            loss = step(stage_x[s], stage_r[s])
            done[s].record()
            loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_loop(max(2, args.warmup))
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    e2e_loop(args.steps)
    t1.record()
    barrier()
    ms_e2e = t0.elapsed_time(t1) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([ms_dev, ms_e2e], device=dev)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = float(times[0]), float(times[1])
    if rank != 0:
        return
    tokens = B * Lq * world
    peak, peak_kind = measured_peaks()
    fwd_ms, bwd_ms = timer.mean_ms("scan_fwd"), timer.mean_ms("scan_bwd")
    bwd_bytes, fwd_bytes = scan_bytes(cfg, B, True), scan_bytes(cfg, B, False)
    achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    per_step_launches = timer.launches / max(1, args.steps) + sum(counted.values())
    line = {
        "metric": "tokens_per_s", "value": tokens / (ms_dev * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 I/O, fp32 state", "data": "synthetic (seeded N(0,1) activations, random-init weights)",
        "config": {"workload": f"mamba1_block fwd+bwd: batch {B}/GPU, seqlen 4096, d_model 768, d_inner 1536, d_state 16, d_conv 4, "
                               "dt_rank 48, RMSNorm eps 1e-5", "parallelism": f"dp{world} (batch replicas, no collective)",
                   "l2": "per-step working set (>1 GB) exceeds the 126 MB L2; inputs alternate between two buffers"},
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4},
        "gpu_launches": int(round(per_step_launches * args.steps)),
        "roofline": {"kernel": "scan_bwd_kernel", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": peak_kind,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch captured with ncu at batch 2
                     # (profiles/scan_kernels_ncu_batch2.md: 127.68 + 44.90 MB), scaled by the batch ratio
                     "traffic": 172.58e6 * B / 2, "bytes_per_launch": bwd_bytes, "ms_per_launch": bwd_ms,
                     "note": "instruction/latency-bound kernel (one ex2 and ~34 warp instructions per 32 (row,state,step)); not HBM-bound on this part"},
        "kernels": {"scan_fwd_kernel": {"ms_per_launch": fwd_ms, "bytes_per_launch": fwd_bytes,
                                        "achieved_gbs": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak}},
        "clocks": clocks,
    }
    if not args.no_cpu and world >= 1:
        line["cpu_baseline"] = cpu_baseline(budget_s=args.cpu_seconds)
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# CPU arm: the oracle (a port of the upstream Python operators) on the host cores
# --------------------------------------------------------------------------------------
def cpu_baseline(budget_s=15.0, steps=None):
    from oracle import ssm_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = dict(CFG, batch=1, seqlen=512)
    w = make_weights(cfg, "cpu", torch.float32, seed=0)
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(cfg["batch"], cfg["seqlen"], cfg["d_model"], generator=g)
    r = torch.randn(cfg["batch"], cfg["seqlen"], cfg["d_model"], generator=g)

    def step():
        for p in w.values():
            p.grad = None
        y, nr = block_forward(orc, w, cfg, x, r)
        (y.float().square().mean() + nr.square().mean() * 1e-3).backward()

    step()  # warm-up
    n, t0 = 0, time.perf_counter()
    while True:
        step()
        n += 1
        el = time.perf_counter() - t0
        if (steps is not None and n >= steps) or (steps is None and (el > budget_s or n >= 50)):
            break
    tok = cfg["batch"] * cfg["seqlen"] * n / el
    return {"value": tok, "unit": "tokens/s", "cores": cores, "kind": "port", "seconds": el,
            "sample": f"same block fwd+bwd at batch 1, seqlen 512 (fp32), {n} passes; upstream's CPU path is its per-token Python loop, "
                      "restated in oracle/ssm_oracle.py"}


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    t0 = time.perf_counter()
    base = cpu_baseline(steps=max(1, args.steps))
    ms = (time.perf_counter() - t0) * 1e3 / max(1, args.steps)
    line = {
        "impl": "reference", "metric": "tokens_per_s", "value": base["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic (seeded)", "config": {"workload": "mamba1_block fwd+bwd (bounded sample: batch 1, seqlen 512)",
                                                 "parallelism": "host cores"},
        "cpu_baseline": base, "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# other workloads of the same hot path (selected with --workload; one JSON line each)
# --------------------------------------------------------------------------------------
def _time_cuda(fn, steps, warmup):
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


def run_ssd(args):
    """BASELINE config 3: Mamba-2 SSD chunk scan, batch 8, L 8192, 48 heads x 64, d_state 128, chunk 256, bf16."""
    from ssm_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, Lq, H, P, N = args.batch or 8, 8192, 48, 64, 128
    g = torch.Generator().manual_seed(0)
    host = dict(
        X=torch.randn(B, Lq, H, P, generator=g).to(torch.bfloat16), dt=(torch.randn(B, Lq, H, generator=g) - 3).to(torch.bfloat16),
        Bm=(torch.randn(B, Lq, 1, N, generator=g) / N ** 0.5).to(torch.bfloat16),
        Cm=(torch.randn(B, Lq, 1, N, generator=g) / N ** 0.5).to(torch.bfloat16), z=torch.randn(B, Lq, H, P, generator=g).to(torch.bfloat16))
    host = {k: v.pin_memory() for k, v in host.items()}
    A = (-torch.exp(torch.rand(H, generator=g) * 2.7726)).to(dev)
    D = torch.randn(H, generator=g).to(dev)
    d = {k: v.to(dev) for k, v in host.items()}

    def step(t):
        return ops.ssd_scan(t["X"], t["dt"], A, t["Bm"], t["Cm"], 256, D=D, z=t["z"], dt_softplus=True, return_final_states=True)

    sampler = ClockSampler(0)
    sampler.start()
    ms = _time_cuda(lambda: step(d), args.steps, args.warmup)
    fin_host = torch.empty(B, H, P, N).pin_memory()
    stage = {k: torch.empty_like(v) for k, v in d.items()}

    def e2e():
        for k in stage:
            stage[k].copy_(host[k], non_blocking=True)
        _, fin = step(stage)
        fin_host.copy_(fin, non_blocking=True)

    ms_e2e = _time_cuda(e2e, max(2, args.steps // 4), 2)
    clocks = sampler.stop()
    peak, kind = measured_peaks()
    io = 2
    bytes_alg = 3 * B * Lq * H * P * io + B * Lq * H * io + 2 * B * Lq * N * io + B * H * P * N * 4 + 2 * H * 4
    flops = B * (Lq // 256) * H * (2 * 256 * 256 * P + 4 * 256 * N * P) + B * (Lq // 256) * 2 * 256 * 256 * N
    tok = B * Lq
    print(json.dumps({
        "metric": "tokens_per_s", "value": tok / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 operands, fp32 accumulate/state",
        "data": "synthetic (seeded)", "config": {"workload": f"ssd chunk scan fwd: batch {B}, seqlen {Lq}, 48 heads x 64, d_state 128, ngroups 1, chunk 256",
                                                 "l2": "inputs (>800 MB) exceed the 126 MB L2"},
        "e2e": {"value": tok / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in host.values()), "d2h_bytes_per_step": fin_host.numel() * 4},
        "gpu_launches": 4 * args.steps,
        "roofline": {"kernel": "ssm_ssd_fwd (cumsum + state + scan kernels)", "bound": "hbm", "achieved": bytes_alg / (ms * 1e-3) / 1e9,
                     "peak": peak, "unit": "GB/s", "frac": bytes_alg / (ms * 1e-3) / 1e9 / peak, "peak_kind": kind, "traffic": None,
                     "bytes_per_launch": bytes_alg, "tensor_tflops": flops / (ms * 1e-3) / 1e12},
        "clocks": clocks}))


def run_decode(args):
    """BASELINE config 4: single-token state steps, batch 256 (a) Mamba-1 layer D 5120, N 16; (b) Mamba-2 state 80 x 64 x 128."""
    from ssm_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(0)
    B, dm, di, n, k, r = 256, 2560, 5120, 16, 4, 160
    bf = torch.bfloat16
    W = {name: (torch.randn(o, i, generator=g) / i ** 0.5).to(bf).to(dev) for name, (o, i) in
         dict(in_proj=(2 * di, dm), x_proj=(r + 2 * n, di), dt_proj=(di, r), out_proj=(dm, di)).items()}
    conv_w = (torch.rand(di, k, generator=g) - 0.5).to(dev)
    A = (-torch.exp(torch.randn(di, n, generator=g) * 0.5)).to(dev)
    Dk, bias = torch.randn(di, generator=g).to(dev), (torch.rand(di, generator=g) * 2 - 4).to(dev)
    ssm_state = (torch.randn(B, di, n, generator=g) * 0.1).to(dev)
    conv_state = (torch.randn(B, di, k, generator=g) * 0.1).to(dev)
    tok = torch.randn(B, dm, generator=g).to(bf).to(dev)

    def layer_step():
        xz = tok @ W["in_proj"].t()
        x, z = xz[:, :di], xz[:, di:]
        u = ops.dw_causal_conv_update(conv_state, x, conv_w, None, "silu")
        xd = u @ W["x_proj"].t()
        delta = xd[:, :r] @ W["dt_proj"].t()
        y = ops.selective_state_step(ssm_state, u, delta, A, xd[:, r:r + n].unsqueeze(1), xd[:, r + n:].unsqueeze(1), D=Dk, z=z,
                                     dt_bias=bias, softplus=True)
        return y @ W["out_proj"].t()

    # (b) Mamba-2 state update alone
    H2, P2, N2 = 80, 64, 128
    st2 = (torch.randn(B, H2, P2, N2, generator=g) * 0.1).to(dev)
    x2, z2 = torch.randn(B, H2, P2, generator=g).to(bf).to(dev), torch.randn(B, H2, P2, generator=g).to(bf).to(dev)
    dt2, A2 = torch.randn(B, H2, generator=g).to(bf).to(dev), (-torch.exp(torch.rand(H2, generator=g))).to(dev)
    B2, C2 = torch.randn(B, 1, N2, generator=g).to(bf).to(dev), torch.randn(B, 1, N2, generator=g).to(bf).to(dev)
    D2 = torch.randn(H2, generator=g).to(dev)

    def m2_step():
        return ops.selective_state_step_heads(st2, x2, dt2, A2, B2, C2, D=D2, z=z2, softplus=True)

    def m1_step_only():
        return ops.selective_state_step(ssm_state, tok[:, :1].expand(B, di).contiguous() if False else x_fixed, d_fixed, A, Bf, Cf, D=Dk, z=z_fixed,
                                        dt_bias=bias, softplus=True)

    x_fixed, d_fixed, z_fixed = (torch.randn(B, di, generator=g).to(bf).to(dev) for _ in range(3))
    Bf, Cf = torch.randn(B, 1, n, generator=g).to(bf).to(dev), torch.randn(B, 1, n, generator=g).to(bf).to(dev)
    steps = max(args.steps, 1000) if args.steps == 20 else args.steps
    sampler = ClockSampler(0)
    sampler.start()
    ms_layer = _time_cuda(layer_step, steps, 20)
    ms_m1 = _time_cuda(m1_step_only, steps, 20)
    ms_m2 = _time_cuda(m2_step, min(steps, 200), 5)
    # CUDA-graph replay of the whole layer step
    graph_ms = None
    try:
        gph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                layer_step()
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(gph):
            out = layer_step()
        graph_ms = _time_cuda(gph.replay, steps, 20)
    except Exception as exc:  # noqa: BLE001
        graph_ms = f"capture failed: {exc}"
    clocks = sampler.stop()
    peak, kind = measured_peaks()
    m1_bytes = 2 * B * di * n * 4 + 4 * B * di * 2 + 2 * B * n * 2 + di * n * 4
    m2_bytes = 2 * B * H2 * P2 * N2 * 4 + 3 * B * H2 * P2 * 2
    val = graph_ms if isinstance(graph_ms, float) else ms_layer
    print(json.dumps({
        "metric": "decode_step_us", "value": val * 1e3, "unit": "us/step", "n_gpus": 1, "steps": steps, "warmup": 20,
        "ms_per_step": val, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations, fp32 state",
        "data": "synthetic (seeded)", "config": {"workload": "decode: Mamba-1 layer step, batch 256, d_model 2560, d_inner 5120, d_state 16, conv 4, dt_rank 160; "
                                                 "1000 consecutive steps", "l2": "state (84 MB) + weights exceed nothing; consecutive dependent steps"},
        "layer_step_us": {"eager": ms_layer * 1e3, "cuda_graph": graph_ms * 1e3 if isinstance(graph_ms, float) else graph_ms},
        "gpu_launches": 2 * steps,
        "roofline": {"kernel": "step_fwd_kernel (Mamba-1 state 256x5120x16)", "bound": "hbm", "achieved": m1_bytes / (ms_m1 * 1e-3) / 1e9, "peak": peak,
                     "unit": "GB/s", "frac": m1_bytes / (ms_m1 * 1e-3) / 1e9 / peak, "peak_kind": kind, "traffic": None, "us_per_launch": ms_m1 * 1e3,
                     "note": "eager launch through ctypes; the 84 MB state stays L2-resident between steps, so this can exceed the HBM peak"},
        "mamba2_state_step": {"us_per_launch": ms_m2 * 1e3, "bytes_per_launch": m2_bytes, "achieved_gbs": m2_bytes / (ms_m2 * 1e-3) / 1e9,
                              "frac": m2_bytes / (ms_m2 * 1e-3) / 1e9 / peak},
        "clocks": clocks}))


def run_scan_c1(args):
    """BASELINE config 1: selective_scan forward, batch 1, D 512, L 2048, N 16, fp32, gated, skip, softplus, last state."""
    from ssm_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    nb, nd, nl, nn = 1, 512, 2048, 16
    # rotate over enough distinct input sets to exceed the L2
    nsets = 10
    sets = []
    for _ in range(nsets):
        sets.append(dict(u=torch.randn(nb, nd, nl), delta=torch.nn.functional.softplus(torch.randn(nb, nd, nl) - 2),
                         B=torch.randn(nb, 1, nn, nl), C=torch.randn(nb, 1, nn, nl), z=torch.randn(nb, nd, nl)))
    A, D = -torch.exp(torch.randn(nd, nn) * 0.5), torch.randn(nd)
    dsets = [{k: v.to(dev) for k, v in s.items()} for s in sets]
    Ad, Dd = A.to(dev), D.to(dev)
    it = [0]

    def step():
        s = dsets[it[0] % nsets]
        it[0] += 1
        return ops.selective_scan(s["u"], s["delta"], Ad, s["B"], s["C"], D=Dd, z=s["z"], softplus=True, return_last_state=True)

    ms = _time_cuda(step, max(args.steps, 50), 10)
    peak, kind = measured_peaks()
    by = 3 * nb * nd * nl * 4 + 2 * nb * nn * nl * 4 + nd * nn * 4 + nd * 4 + nb * nd * nl * 4 + nb * nd * nn * 4
    from oracle import ssm_oracle as orc

    torch.set_num_threads(os.cpu_count() or 1)
    s0 = sets[0]
    t0 = time.perf_counter()
    orc.selective_scan(s0["u"], s0["delta"], A, s0["B"], s0["C"], D=D, z=s0["z"], softplus=True, return_last_state=True)
    cpu_s = time.perf_counter() - t0
    print(json.dumps({
        "metric": "tokens_per_s", "value": nb * nl / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": max(args.steps, 50), "warmup": 10,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic (seeded)",
        "config": {"workload": "selective_scan fwd: batch 1, d_inner 512, seqlen 2048, d_state 16, fp32 (README prefill_2k_d512)",
                   "l2": "10 rotating input sets (171 MB) exceed the 126 MB L2"},
        "gpu_launches": max(args.steps, 50),
        "roofline": {"kernel": "scan_fwd_kernel", "bound": "hbm", "achieved": by / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": by / (ms * 1e-3) / 1e9 / peak, "peak_kind": kind, "traffic": None, "bytes_per_launch": by},
        "cpu_baseline": {"value": nb * nl / cpu_s, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port", "seconds": cpu_s,
                         "sample": "the full config once (upstream README reports 1012.9 ms for its Python backend)"}}))


def run_ssd_sp(args):
    """Long-sequence Mamba-2 SSD core, sequence-sharded (BASELINE config 5's per-layer scan): batch 2, seqlen 131072
    split into contiguous shards over the ranks, 80 heads x 64, d_state 128, chunk 256; strong scaling."""
    import torch.distributed as dist

    from ssm_b200 import seqpar

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    under_launcher = "RANK" in os.environ
    if under_launcher:
        dist.init_process_group("nccl", device_id=dev)
    B, Ltot, H, P, N = 2, args.seqlen or 131072, 80, 64, 128
    Lq = Ltot // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)  # generated on the device: the shard is several GB
    bf = torch.bfloat16
    X = torch.randn(B, Lq, H, P, generator=g, device=dev, dtype=bf)
    z = torch.randn(B, Lq, H, P, generator=g, device=dev, dtype=bf)
    dt = (torch.randn(B, Lq, H, generator=g, device=dev) - 3).to(bf)
    Bm = (torch.randn(B, Lq, 1, N, generator=g, device=dev) / N ** 0.5).to(bf)
    Cm = (torch.randn(B, Lq, 1, N, generator=g, device=dev) / N ** 0.5).to(bf)
    if rank == 0:
        print(f"[ssd_sp] inputs ready: shard length {Lq}", file=sys.stderr, flush=True)
    g0 = torch.Generator().manual_seed(7)
    A = (-torch.exp(torch.rand(H, generator=g0) * 2.7726)).to(dev)
    D = torch.randn(H, generator=g0).to(dev)

    def step():
        return seqpar.ssd_scan_sharded(X, dt, A, Bm, Cm, 256, D=D, z=z, dt_softplus=True)

    tw = time.perf_counter()
    for i in range(args.warmup):
        step()
        torch.cuda.synchronize()
        if rank == 0:
            print(f"[ssd_sp] warm-up {i}: {time.perf_counter() - tw:.3f} s since start", file=sys.stderr, flush=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        ms = float(t[0])
        peak, kind = measured_peaks()
        bytes_alg = (3 * B * Ltot * H * P * 2 + B * Ltot * H * 2 + 2 * B * Ltot * N * 2) / world  # per GPU
        print(json.dumps({
            "metric": "tokens_per_s", "value": B * Ltot / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 operands, fp32 accumulate/state", "data": "synthetic (seeded)",
            "config": {"workload": f"sequence-sharded ssd scan: batch {B}, seqlen {Ltot} in {world} contiguous shards, 80 heads x 64, d_state 128, chunk 256",
                       "parallelism": f"sp{world}: all-gather of (final state 5.2 MB, log-decay) per rank over NCCL, associative fold",
                       "l2": "per-GPU inputs exceed the 126 MB L2"},
            "gpu_launches": 5 * args.steps,
            "roofline": {"kernel": "ssm_ssd_fwd phases 1+2 per shard", "bound": "hbm", "achieved": bytes_alg / (ms * 1e-3) / 1e9, "peak": peak,
                         "unit": "GB/s", "frac": bytes_alg / (ms * 1e-3) / 1e9 / peak, "peak_kind": kind, "traffic": None},
            "clocks": clocks}))
    if under_launcher:
        dist.destroy_process_group()


def run_mamba2_sp(args):
    """BASELINE config 5: a random-init bf16 Mamba-2 stack (d_model 2560, expand 2, headdim 64, d_state 128, ngroups 1,
    chunk 256, conv width 4, RMSNorm, vocab 50280 with a tied head) prefilling batch 2 x seqlen 131072 of uniform random
    token ids, the sequence split into contiguous shards over the ranks: per layer the K-1 trailing conv inputs go to
    the next rank and the chunk state is handed over (`ssm_b200.seqpar`).  A step is one whole forward; the result is
    the logits of the last token (on the last rank)."""
    import torch.distributed as dist

    from ssm_b200 import ops
    from ssm_b200.mixer import mamba2_block_forward

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    under_launcher = "RANK" in os.environ
    if under_launcher:
        dist.init_process_group("nccl", device_id=dev)
    B, Ltot = 2, args.seqlen or 131072
    layers = args.layers or 64
    dm, hp, n, k, vocab = 2560, 64, 128, 4, 50280
    di = 2 * dm
    nh = di // hp
    Lq = Ltot // world
    bf = torch.bfloat16
    cfg = dict(heads=nh, headdim=hp, d_state=n, groups=1, chunk_size=256, eps=1e-5)
    gen = torch.Generator(device=dev).manual_seed(1234)  # the same weights on every rank

    def lin(o, i):
        return (torch.randn(o, i, generator=gen, device=dev) / i ** 0.5).to(bf)

    def layer_weights():
        return dict(
            pre_norm_w=torch.ones(dm, device=dev, dtype=bf), in_z=lin(di, dm), in_x=lin(di, dm), in_B=lin(n, dm), in_C=lin(n, dm), in_dt=lin(nh, dm),
            conv_x=(torch.rand(di, k, generator=gen, device=dev) - 0.5).to(bf), conv_B=(torch.rand(n, k, generator=gen, device=dev) - 0.5).to(bf),
            conv_C=(torch.rand(n, k, generator=gen, device=dev) - 0.5).to(bf), conv_x_b=torch.zeros(di, device=dev, dtype=bf),
            conv_B_b=torch.zeros(n, device=dev, dtype=bf), conv_C_b=torch.zeros(n, device=dev, dtype=bf),
            dt_bias=(torch.rand(nh, generator=gen, device=dev) * 2 - 4).float(), A_log=torch.log(torch.rand(nh, generator=gen, device=dev) * 15 + 1),
            D=torch.randn(nh, generator=gen, device=dev), norm_w=torch.ones(di, device=dev, dtype=bf), out_proj=lin(dm, di))

    ws = [layer_weights() for _ in range(layers)]
    emb = (torch.randn(vocab, dm, generator=gen, device=dev) * 0.02).to(bf)
    final_norm = torch.ones(dm, device=dev, dtype=bf)
    gi = torch.Generator().manual_seed(99)
    ids_all = torch.randint(0, vocab, (B, Ltot), generator=gi)
    ids_host = ids_all[:, rank * Lq:(rank + 1) * Lq].contiguous().pin_memory()
    if rank == 0:
        print(f"[mamba2_sp] {layers} layers ready: shard length {Lq}", file=sys.stderr, flush=True)

    @torch.no_grad()
    def forward(ids):
        hidden = torch.nn.functional.embedding(ids, emb)
        residual = None
        for w in ws:
            hidden, residual = mamba2_block_forward(ops, w, cfg, hidden, residual, sharded=world > 1)
        last = ops.fused_layer_norm(hidden[:, -1:].contiguous(), final_norm, None, residual=residual[:, -1:].contiguous(), is_rms=True, eps=1e-5,
                                    prenorm=True, residual_in_fp32=True)
        return torch.matmul(last[:, 0], emb.t())  # logits of the shard's last token; the sequence's last token on the last rank

    ids_dev = ids_host.to(dev)
    tw = time.perf_counter()
    for i in range(args.warmup):
        forward(ids_dev)
        torch.cuda.synchronize()
        if rank == 0:
            print(f"[mamba2_sp] warm-up {i}: {time.perf_counter() - tw:.2f} s since start", file=sys.stderr, flush=True)

    def timed(fn):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(lambda: forward(ids_dev))
    clocks = sampler.stop() if rank == 0 else None
    out_host = torch.empty(B, vocab, dtype=bf).pin_memory()

    def e2e_step():
        logits = forward(ids_host.to(dev, non_blocking=True))
        out_host.copy_(logits, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    ms_e2e = timed(e2e_step)
    if rank == 0:
        tokens = B * Ltot
        gemm_flops = 2.0 * tokens * dm * (2 * di + 2 * n + nh + di) * layers
        print(json.dumps({
            "metric": "tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 weights / activations, fp32 residual stream and states", "data": "synthetic (seeded uniform token ids, random-init weights)",
            "config": {"workload": f"mamba2 prefill: {layers} layers, d_model {dm}, {nh} heads x {hp}, d_state {n}, chunk 256, conv {k}, vocab {vocab}; "
                                   f"batch {B}, seqlen {Ltot} in {world} contiguous shards",
                       "parallelism": f"sp{world}: per layer a {k - 1}-token conv halo to the next rank and an all-gather of the chunk state (5.2 MB / rank)",
                       "l2": "per-layer activations (GBs) exceed the 126 MB L2"},
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": ids_host.numel() * 8,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": layers * 9 * args.steps,
            "roofline": {"kernel": "whole forward (projection GEMMs dominate)", "bound": "tensor", "achieved": gemm_flops / (ms * 1e-3) / 1e12 / world,
                         "peak": None, "unit": "TFLOP/s", "frac": None, "traffic": None, "note": "dense projection flops per GPU over the whole step"},
            "clocks": clocks}))
    if under_launcher:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (profiling on a smaller case)")
    ap.add_argument("--workload", default="mamba1_block", choices=["mamba1_block", "ssd", "decode", "scan_c1", "ssd_sp", "mamba2_sp"])
    ap.add_argument("--layers", type=int, default=0, help="override the depth of the mamba2_sp workload")
    ap.add_argument("--seqlen", type=int, default=0, help="override the total sequence length of the ssd_sp workload")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "ssd":
        run_ssd(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.workload == "scan_c1":
        run_scan_c1(args)
    elif args.workload == "mamba2_sp":
        run_mamba2_sp(args)
    elif args.workload == "ssd_sp":
        run_ssd_sp(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
