"""`ssm_b200.lm` on the CPU oracle namespace: the wrapper's own logic (fused add + norm chaining, decode caches,
greedy generation, configuration surface) without a GPU."""

from __future__ import annotations

import pytest
import torch

from oracle import ssm_oracle as orc
from ssm_b200.lm import MambaConfig, MambaLMHeadModel, MixerModel

KINDS = [("Mamba1", dict(d_state=8)), ("Mamba2", dict(d_state=16, headdim=8))]


@pytest.mark.parametrize("kind,extra", KINDS, ids=[k for k, _ in KINDS])
def test_token_by_token_decode_reproduces_the_full_forward(kind, extra):
    torch.manual_seed(0)
    cfg = MambaConfig(d_model=32, n_layer=3, vocab_size=50, ssm_cfg=dict(layer=kind, **extra))
    model = MambaLMHeadModel(cfg, ops=orc)
    assert model.lm_head.weight is model.backbone.embedding.weight and model.lm_head.weight.shape[0] == 56  # padded to a multiple of 8, tied
    ids = torch.randint(0, 50, (2, 9))
    with torch.no_grad():
        full = model(ids).logits
        cache = model.allocate_inference_cache(2, max_seqlen=9)
        steps = torch.cat([model(ids[:, t:t + 1], inference_params=cache).logits for t in range(9)], dim=1)
        assert cache.seqlen_offset == 9
        torch.testing.assert_close(steps, full, rtol=1e-4, atol=1e-5)
        assert model(ids, num_last_tokens=2).logits.shape == (2, 2, 56)
        out = model.generate(ids[:, :4], 8)
    assert out.shape == (2, 8) and torch.equal(out[:, :4], ids[:, :4])
    # greedy continuation = argmax of the full forward on the generated prefix
    with torch.no_grad():
        again = model(out[:, :-1]).logits.argmax(-1)
    assert torch.equal(again[:, 3:], out[:, 4:])


def test_layer_is_upstreams_fused_add_norm_block():
    """hidden, residual = norm(hidden + residual), hidden + residual; then the mixer (src/ssm/modules/block.py:109-131)."""
    torch.manual_seed(1)
    model = MixerModel(d_model=16, n_layer=2, d_intermediate=0, vocab_size=20, ssm_cfg=dict(layer="Mamba1", d_state=4), rms_norm=True,
                       residual_in_fp32=True, ops=orc)
    ids = torch.randint(0, 20, (1, 5))
    with torch.no_grad():
        got = model(ids)
        hidden, residual = model.embedding(ids), None
        for layer in model.layers:
            residual = hidden.float() if residual is None else hidden.float() + residual
            normed = residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + 1e-5) * layer.norm_w
            hidden = layer.mixer_forward(normed)
        residual = hidden.float() + residual
        want = residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + 1e-5) * model.norm_f_weight
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)


def test_gradients_reach_every_layer_through_the_residual_stream():
    torch.manual_seed(2)
    model = MambaLMHeadModel(MambaConfig(d_model=16, n_layer=3, vocab_size=24, ssm_cfg=dict(layer="Mamba1", d_state=4)), ops=orc)
    model(torch.randint(0, 24, (2, 6))).logits.square().mean().backward()
    for i, layer in enumerate(model.backbone.layers):
        for name in ("in_x", "out_proj", "norm_w", "A_log"):
            g = getattr(layer, name).grad
            assert g is not None and float(g.abs().max()) > 0, f"layer {i} {name}"


def test_configuration_surface_and_rejections():
    cfg = MambaConfig()
    assert (cfg.d_model, cfg.n_layer, cfg.vocab_size, cfg.rms_norm, cfg.fused_add_norm, cfg.residual_in_fp32, cfg.tie_embeddings) == \
        (2560, 64, 50277, True, True, True, True)
    with pytest.raises(ValueError):
        MixerModel(d_model=8, n_layer=1, d_intermediate=0, vocab_size=8, attn_layer_idx=[0])
    with pytest.raises(ValueError):
        MixerModel(d_model=8, n_layer=1, d_intermediate=16, vocab_size=8)
    with pytest.raises(ValueError):
        MixerModel(d_model=8, n_layer=1, d_intermediate=0, vocab_size=8, ssm_cfg=dict(layer="S4"))
    model = MambaLMHeadModel(MambaConfig(d_model=8, n_layer=1, vocab_size=8, ssm_cfg=dict(layer="Mamba1", d_state=2)), ops=orc)
    with pytest.raises(ValueError):
        model(torch.zeros(8, dtype=torch.long))
    # LayerNorm flavour: a bias per norm
    ln = MixerModel(d_model=8, n_layer=1, d_intermediate=0, vocab_size=8, ssm_cfg=dict(layer="Mamba1", d_state=2), rms_norm=False, ops=orc)
    assert ln.norm_f_bias is not None and ln(torch.zeros(1, 3, dtype=torch.long)).shape == (1, 3, 8)
