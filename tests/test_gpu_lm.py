"""`ssm_b200.lm` on the CUDA operators against the same model on the CPU oracle: logits, decode caches, greedy
generation eager and under CUDA-graph replay."""

from __future__ import annotations

import copy

import pytest
import torch

from oracle import ssm_oracle as orc
from tests.gpu_util import close

pytestmark = pytest.mark.gpu


def _pair(kind, **extra):
    from ssm_b200.lm import MambaConfig, MambaLMHeadModel

    torch.manual_seed(5)
    cfg = MambaConfig(d_model=128, n_layer=2, vocab_size=96, ssm_cfg=dict(layer=kind, **extra))
    cpu = MambaLMHeadModel(cfg, ops=orc)
    gpu = MambaLMHeadModel(cfg)
    gpu.load_state_dict(copy.deepcopy(cpu.state_dict()))
    return cpu, gpu.cuda()


@pytest.mark.parametrize("kind,extra", [("Mamba1", dict(d_state=16)), ("Mamba2", dict(d_state=128, headdim=64))], ids=["Mamba1", "Mamba2"])
def test_lm_matches_oracle_and_decodes(kind, extra):
    cpu, gpu = _pair(kind, **extra)
    if kind == "Mamba2":  # the tensor-core scan takes 16-bit operands
        for name, p in gpu.named_parameters():
            if not any(k in name for k in ("dt_bias", "A_log", ".D")):
                p.data = p.data.to(torch.bfloat16)
        for (name, pc), (_, pg) in zip(cpu.named_parameters(), gpu.named_parameters()):
            pc.data = pg.data.float().cpu()
    ids = torch.randint(0, 96, (2, 300))
    tol = dict(rtol=1e-4, atol=1e-5) if kind == "Mamba1" else dict(rtol=2e-2, atol=2e-2)
    with torch.no_grad():
        want = cpu(ids).logits
        got = gpu(ids.cuda()).logits
        close(got, want, **tol, what="logits", reduced=True)
        # token-by-token decode reproduces the prefill
        cache = gpu.allocate_inference_cache(2)
        steps = torch.cat([gpu(ids[:, t:t + 1].cuda(), inference_params=cache).logits for t in range(24)], dim=1)
        close(steps, got[:, :24], **tol, what="decode vs prefill", reduced=True)
        eager = gpu.generate(ids[:, :5].cuda(), 16)
        graphed = gpu.generate(ids[:, :5].cuda(), 16, cuda_graph=True)
    assert eager.shape == (2, 16) and torch.equal(eager, graphed)
