"""`ssm_b200.mixer.Mamba1Block` on the CUDA operators against the same block on the CPU oracle.

A block chains the operators with cuBLAS projections, so every compared tensor is a contraction
over hundreds of terms: the absolute term of the bar is scaled by the tensor's magnitude (``reduced=True``)."""

from __future__ import annotations

import copy

import pytest
import torch

from oracle import ssm_oracle as orc
from tests.gpu_util import FP32_TOL, close

HALF_TOL = dict(rtol=2e-2, atol=2e-2)

pytestmark = pytest.mark.gpu


def _pair(d_model, dtype, **kw):
    from ssm_b200.mixer import Mamba1Block

    torch.manual_seed(d_model)
    cpu = Mamba1Block(d_model, ops=orc, **kw)
    gpu = Mamba1Block(d_model, **kw)  # ops=None: the CUDA operators
    gpu.load_state_dict(copy.deepcopy(cpu.state_dict()))
    gpu = gpu.cuda()
    if dtype != torch.float32:
        for name in ("in_x", "in_z", "conv_w", "conv_b", "x_proj", "dt_proj", "out_proj", "norm_w"):
            p = getattr(gpu, name)
            p.data = p.data.to(dtype)
            getattr(cpu, name).data = p.data.float().cpu()  # the oracle block computes in fp32 from the rounded weights
    return cpu, gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_forward_backward_match_oracle(dtype):
    cpu, gpu = _pair(64, dtype, d_state=16, d_conv=4, expand=2)
    gen = torch.Generator().manual_seed(3)
    hidden = torch.randn(2, 160, 64, generator=gen).to(dtype)
    residual = torch.randn(2, 160, 64, generator=gen)
    ho = hidden.float().clone().requires_grad_(True)
    hg = hidden.cuda().requires_grad_(True)
    yo, ro = cpu(ho, residual)
    yg, rg = gpu(hg, residual.cuda())
    tol = FP32_TOL if dtype == torch.float32 else HALF_TOL
    close(yg, yo, **tol, what="normed output", reduced=True)
    close(rg, ro, **tol, what="residual stream", reduced=True)
    wy = torch.randn(yo.shape, generator=gen).to(dtype).float()
    names = ["x_proj", "dt_proj", "A_log", "dt_bias", "D", "conv_w", "out_proj"]
    go = torch.autograd.grad((yo * wy).sum(), [ho] + [getattr(cpu, n) for n in names])
    gg = torch.autograd.grad((yg.float() * wy.cuda()).sum(), [hg] + [getattr(gpu, n) for n in names])
    for name, a, b in zip(["hidden"] + names, gg, go):
        close(a, b, **tol, what=f"grad {name}", reduced=True)


def test_step_reproduces_forward_and_replays_under_a_cuda_graph():
    cpu, gpu = _pair(48, torch.float32, d_state=8, d_conv=4, expand=2)
    del cpu
    torch.manual_seed(7)
    hidden = torch.randn(4, 9, 48, device="cuda")
    residual = torch.randn(4, 9, 48, device="cuda")
    with torch.no_grad():
        y, r = gpu(hidden, residual)
        conv_state, ssm_state = gpu.allocate_inference_cache(4)
        for t in range(9):
            yt, rt = gpu.step(hidden[:, t:t + 1].contiguous(), residual[:, t:t + 1].contiguous(), conv_state, ssm_state)
            close(yt, y[:, t:t + 1], **FP32_TOL, what=f"step {t}", reduced=True)
            close(rt, r[:, t:t + 1], **FP32_TOL, what=f"residual {t}", reduced=True)
        # the same nine steps as graph replays of one captured step
        conv2, ssm2 = gpu.allocate_inference_cache(4)
        tok, res = torch.zeros(4, 1, 48, device="cuda"), torch.zeros(4, 1, 48, device="cuda")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up outside capture (allocator, lazy library state)
                gpu.step(tok, res, conv2.clone(), ssm2.clone())
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out_y, out_r = gpu.step(tok, res, conv2, ssm2)
        conv2.zero_(), ssm2.zero_()
        for t in range(9):
            tok.copy_(hidden[:, t:t + 1]), res.copy_(residual[:, t:t + 1])
            graph.replay()
            close(out_y, y[:, t:t + 1], **FP32_TOL, what=f"graph step {t}", reduced=True)
    close(ssm2, ssm_state, **FP32_TOL, what="state after nine graph replays", reduced=True)


def test_mamba2_block_matches_oracle_and_the_sharded_path_agrees():
    """Tensor-core shape (headdim 64, d_state 128, bf16): block output against the fp32 oracle block, and the
    two-phase (sequence-shard) execution of the same block on a single rank against the direct one."""
    from ssm_b200.mixer import Mamba2Block

    torch.manual_seed(11)
    cpu = Mamba2Block(128, d_state=128, headdim=64, expand=2, ops=orc)
    gpu = Mamba2Block(128, d_state=128, headdim=64, expand=2)
    gpu.load_state_dict(copy.deepcopy(cpu.state_dict()))
    gpu = gpu.cuda()
    for name, p in gpu.named_parameters():
        if name not in ("dt_bias", "A_log", "D"):
            p.data = p.data.to(torch.bfloat16)
            dict(cpu.named_parameters())[name].data = p.data.float().cpu()
    hidden = torch.randn(2, 600, 128).to(torch.bfloat16)
    residual = torch.randn(2, 600, 128)
    with torch.no_grad():
        yo, ro = cpu(hidden.float(), residual)
        yg, rg = gpu(hidden.cuda(), residual.cuda())
        ys, rs = gpu(hidden.cuda(), residual.cuda(), sharded=True)
    close(rg, ro, **HALF_TOL, what="residual stream", reduced=True)
    close(yg, yo, **HALF_TOL, what="block output", reduced=True)
    close(ys, yg, **HALF_TOL, what="two-phase execution", reduced=True)
    assert torch.equal(rs, rg)


def test_two_stacked_blocks_pass_gradients_through_the_residual_stream():
    """The residual stream a block returns is an input of the next block: its gradient has to reach the first
    block's parameters and input.  Loss terms on both the last normed output and the last residual."""
    c1, g1 = _pair(64, torch.float32, d_state=16, d_conv=4, expand=2)
    c2, g2 = _pair(64, torch.float32, d_state=16, d_conv=4, expand=2)
    gen = torch.Generator().manual_seed(9)
    hidden, residual = torch.randn(2, 96, 64, generator=gen), torch.randn(2, 96, 64, generator=gen)
    wy, wr = torch.randn(2, 96, 64, generator=gen), torch.randn(2, 96, 64, generator=gen)
    ho, ro = hidden.clone().requires_grad_(True), residual.clone().requires_grad_(True)
    hg, rg = hidden.cuda().requires_grad_(True), residual.cuda().requires_grad_(True)

    def run(b1, b2, h, r, dev):
        y1, r1 = b1(h, r)
        y2, r2 = b2(y1, r1)
        return y2, r2, (y2 * wy.to(dev)).sum() + (r2 * wr.to(dev)).sum()

    yo, r2o, lo = run(c1, c2, ho, ro, "cpu")
    yg, r2g, lg = run(g1, g2, hg, rg, "cuda")
    close(yg, yo, **FP32_TOL, what="normed output", reduced=True)
    close(r2g, r2o, **FP32_TOL, what="residual stream", reduced=True)
    names = ["in_x", "x_proj", "A_log", "D", "out_proj", "norm_w"]
    go = torch.autograd.grad(lo, [ho, ro] + [getattr(c1, n) for n in names])
    gg = torch.autograd.grad(lg, [hg, rg] + [getattr(g1, n) for n in names])
    for name, a, b in zip(["hidden", "residual"] + names, gg, go):
        close(a, b, **FP32_TOL, what=f"grad {name} of the first block", reduced=True)
