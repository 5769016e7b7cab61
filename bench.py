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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
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


def block_forward(ops, w, cfg, hidden, residual):
    """hidden (B, L, d_model) activations, residual (B, L, d_model) fp32 stream -> (normed, new_residual)."""
    n, r = cfg["d_state"], cfg["dt_rank"]
    ht = hidden.transpose(1, 2)
    x = torch.matmul(w["in_x"], ht)                                    # (B, Di, L): the two halves of in_proj
    z = torch.matmul(w["in_z"], ht)
    u = ops.dw_causal_conv(x, w["conv_w"], w["conv_b"], "silu")
    x_dbl = torch.matmul(w["x_proj"], u)                               # (B, R + 2N, L)
    dt_low, Bm, Cm = torch.split(x_dbl, [r, n, n], dim=1)
    delta = torch.matmul(w["dt_proj"], dt_low)                         # (B, Di, L)
    y = ops.selective_scan(u, delta, w["A"], Bm.unsqueeze(1), Cm.unsqueeze(1), D=w["D"], z=z, dt_bias=w["dt_bias"], softplus=True)
    out = torch.matmul(y.transpose(1, 2), w["out_proj"].t())          # (B, L, d_model)
    return ops.fused_layer_norm(out, w["norm_w"], None, residual=residual, is_rms=True, eps=1e-5, prenorm=True,
                                residual_in_fp32=True, return_residual=True)


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
                     "frac": achieved / peak, "peak_kind": peak_kind, "traffic": None, "bytes_per_launch": bwd_bytes,
                     "ms_per_launch": bwd_ms},
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (profiling on a smaller case)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
