"""Language-model wrapper on the B200 operators: ``MixerModel`` / ``MambaLMHeadModel`` with the constructor and
call signatures of the upstream classes (src/ssm/models/lm.py:175-392, 395-520; configuration
src/ssm/models/config.py), built from this package's mixer blocks.

Every layer is upstream's fused-add-norm block (src/ssm/modules/block.py:109-131): ``residual = hidden + residual``
and ``hidden = norm(residual)`` are ONE call of ``fused_layer_norm(..., return_residual=True)`` (upstream routes that
to an external Triton kernel), followed by the mixer; the final norm folds the last residual add the same way
(lm.py:378-387).  The residual stream is kept in fp32 when ``residual_in_fp32``.  Mixers: ``ssm_cfg["layer"]`` selects
``"Mamba1"`` (selective scan) or ``"Mamba2"`` (state-space-dual scan with a d_state axis, upstream Mamba-2 layout).
Attention layers and the gated MLP of upstream's hybrid configurations are outside the operator hot path and are
rejected.  Beyond upstream: ``forward(..., sharded=True, group=pg)`` runs a Mamba-2 stack on one contiguous shard of a
sequence split over ranks (`ssm_b200.seqpar`), and ``step`` decodes one token against caches allocated by
``allocate_inference_cache``.
"""

from __future__ import annotations

from collections import namedtuple
from dataclasses import dataclass, field
from typing import Any, Optional

import torch
from torch import Tensor, nn

from .mixer import Mamba1Block, Mamba2Block

CausalLMOutput = namedtuple("CausalLMOutput", ["logits"])


def _default_ssm_cfg() -> dict:
    return {"layer": "Mamba1", "dt_rank": "auto", "dt_min": 1e-3, "dt_max": 1e-1, "dt_init_floor": 1e-4}


@dataclass
class MambaConfig:
    """Same fields and defaults as upstream's ``MambaConfig`` (src/ssm/models/config.py)."""

    d_model: int = 2560
    d_intermediate: int = 0
    n_layer: int = 64
    vocab_size: int = 50277
    ssm_cfg: dict = field(default_factory=_default_ssm_cfg)
    attn_layer_idx: list = field(default_factory=list)
    attn_cfg: dict = field(default_factory=dict)
    rms_norm: bool = True
    residual_in_fp32: bool = True
    fused_add_norm: bool = True
    pad_vocab_size_multiple: int = 8
    tie_embeddings: bool = True


@dataclass
class InferenceCache:
    """Per-layer decode state (what upstream keeps in ``InferenceParams.layer_states``)."""

    layer_states: dict
    seqlen_offset: int = 0


class MixerModel(nn.Module):
    """Embedding, ``n_layer`` fused-add-norm mixer blocks, final norm (upstream ``MixerModel``, lm.py:175-392)."""

    def __init__(self, *, d_model: int, n_layer: int, d_intermediate: int, vocab_size: int, ssm_cfg: Optional[dict] = None,
                 attn_layer_idx: Optional[list] = None, attn_cfg: Optional[dict] = None, norm_epsilon: float = 1e-5, rms_norm: bool = False,
                 initializer_cfg: Optional[dict] = None, fused_add_norm: bool = False, residual_in_fp32: bool = False, device=None, dtype=None,
                 ops: Any = None) -> None:
        super().__init__()
        if attn_layer_idx or d_intermediate:
            raise ValueError("attention layers and the gated MLP are not part of the state-space operator path")
        del attn_cfg, fused_add_norm  # the add + norm of every layer always runs as one fused operator call
        cfg = dict(ssm_cfg or {})
        kind = cfg.pop("layer", "Mamba1")
        cfg.pop("dt_init", None)
        if kind == "Mamba2":
            cfg.pop("dt_rank", None)  # Mamba-2 has one step size per head, projected straight from the input
        if kind not in ("Mamba1", "Mamba2"):
            raise ValueError("ssm_cfg['layer'] must be either 'Mamba1' or 'Mamba2'")
        self.kind, self.rms_norm, self.eps, self.residual_in_fp32 = kind, bool(rms_norm), norm_epsilon, bool(residual_in_fp32)
        self.d_model = d_model
        self._ops = ops
        kw = dict(device=device, dtype=dtype)
        self.embedding = nn.Embedding(vocab_size, d_model, **kw)
        std = (initializer_cfg or {}).get("initializer_range", 0.02)
        nn.init.normal_(self.embedding.weight, std=std)
        block = Mamba1Block if kind == "Mamba1" else Mamba2Block
        # a block's own norm weight (`norm_w` / `pre_norm_w`) serves as the pre-norm of its layer
        self.layers = nn.ModuleList([block(d_model, eps=norm_epsilon, ops=ops, **cfg, **kw) for _ in range(n_layer)])
        self.norm_f_weight = nn.Parameter(torch.ones(d_model, **kw))
        self.norm_f_bias = None if rms_norm else nn.Parameter(torch.zeros(d_model, **kw))
        if not rms_norm:
            for layer in self.layers:
                layer.norm_b = nn.Parameter(torch.zeros(d_model, **kw))
        rescale = (initializer_cfg or {}).get("rescale_prenorm_residual", True)
        if rescale:  # upstream divides the output projections by sqrt(n_layer) (lm.py:80-98)
            with torch.no_grad():
                for layer in self.layers:
                    layer.out_proj /= n_layer ** 0.5

    def _namespace(self):
        if self._ops is not None:
            return self._ops
        from . import ops

        return ops

    def _pre_norm(self, layer):
        return (layer.norm_w if self.kind == "Mamba1" else layer.pre_norm_w), getattr(layer, "norm_b", None)

    def allocate_inference_cache(self, batch_size: int, max_seqlen: int = 0, dtype: Optional[torch.dtype] = None, **kwargs) -> InferenceCache:
        del max_seqlen, kwargs  # state-space layers keep a fixed-size state
        return InferenceCache({i: layer.allocate_inference_cache(batch_size, dtype) for i, layer in enumerate(self.layers)})

    def forward(self, input_ids: Tensor, *, inference_params: Optional[InferenceCache] = None, sharded: bool = False, group=None) -> Tensor:
        """``input_ids (B, L)`` -> hidden states ``(B, L, d_model)`` after the final norm.  With ``inference_params`` and
        ``L == 1`` the call advances the caches by one token (decode)."""
        ops = self._namespace()
        hidden = self.embedding(input_ids)
        residual = None
        decode = inference_params is not None and input_ids.shape[1] == 1
        if inference_params is not None and not decode:
            raise ValueError("prefill into a cache is not built: feed the prompt token by token, or run forward() without a cache")
        for i, layer in enumerate(self.layers):
            w, b = self._pre_norm(layer)
            hidden, residual = ops.fused_layer_norm(hidden, w, b, residual=residual, is_rms=self.rms_norm, eps=self.eps, prenorm=True,
                                                    residual_in_fp32=self.residual_in_fp32, return_residual=True)
            if decode:
                hidden = layer.mixer_step(hidden[:, 0], inference_params.layer_states[i]).unsqueeze(1)
            elif self.kind == "Mamba2":
                hidden = layer.mixer_forward(hidden, sharded=sharded, group=group)
            else:
                if sharded:
                    raise ValueError("sequence-sharded prefill is built for Mamba2 layers")
                hidden = layer.mixer_forward(hidden)
        if inference_params is not None:
            inference_params.seqlen_offset += input_ids.shape[1]
        return ops.fused_layer_norm(hidden, self.norm_f_weight, self.norm_f_bias, residual=residual, is_rms=self.rms_norm, eps=self.eps,
                                    prenorm=True, residual_in_fp32=self.residual_in_fp32)


class MambaLMHeadModel(nn.Module):
    """Backbone plus (tied) output head; ``forward`` returns ``CausalLMOutput(logits)`` (upstream lm.py:395-520)."""

    def __init__(self, config: MambaConfig, initializer_cfg: Optional[dict] = None, device=None, dtype=None, ops: Any = None) -> None:
        super().__init__()
        self.config = config
        vocab = config.vocab_size
        if vocab % config.pad_vocab_size_multiple:
            vocab += config.pad_vocab_size_multiple - vocab % config.pad_vocab_size_multiple
        self.backbone = MixerModel(d_model=config.d_model, n_layer=config.n_layer, d_intermediate=config.d_intermediate, vocab_size=vocab,
                                   ssm_cfg=config.ssm_cfg, attn_layer_idx=config.attn_layer_idx, attn_cfg=config.attn_cfg, rms_norm=config.rms_norm,
                                   fused_add_norm=config.fused_add_norm, residual_in_fp32=config.residual_in_fp32, initializer_cfg=initializer_cfg,
                                   device=device, dtype=dtype, ops=ops)
        self.lm_head = nn.Linear(config.d_model, vocab, bias=False, device=device, dtype=dtype)
        self.tie_weights()

    def tie_weights(self) -> None:
        if self.config.tie_embeddings:
            self.lm_head.weight = self.backbone.embedding.weight

    def allocate_inference_cache(self, batch_size: int, max_seqlen: int = 0, dtype: Optional[torch.dtype] = None, **kwargs) -> InferenceCache:
        return self.backbone.allocate_inference_cache(batch_size, max_seqlen, dtype=dtype, **kwargs)

    def forward(self, input_ids: Tensor, position_ids: Optional[Tensor] = None, inference_params: Optional[InferenceCache] = None,
                num_last_tokens: int = 0, **mixer_kwargs) -> CausalLMOutput:
        del position_ids
        if input_ids.dim() != 2:
            raise ValueError("input_ids must be a 2D tensor of shape (batch, seqlen)")
        hidden = self.backbone(input_ids, inference_params=inference_params, **mixer_kwargs)
        if num_last_tokens > 0:
            hidden = hidden[:, -num_last_tokens:, :]
        return CausalLMOutput(logits=self.lm_head(hidden))

    @torch.no_grad()
    def generate(self, input_ids: Tensor, max_length: int, cuda_graph: bool = False) -> Tensor:
        """Greedy decoding: the prompt is fed token by token into fresh caches, then ``max_length - prompt`` tokens are
        produced.  ``cuda_graph=True`` captures one decode step and replays it (what upstream's generation driver does,
        src/ssm/utils/generation.py:187-315)."""
        nb, plen = input_ids.shape
        cache = self.allocate_inference_cache(nb)
        tok = input_ids[:, :1].clone()
        logits = None
        step = lambda: self.forward(tok, inference_params=cache).logits[:, -1]  # noqa: E731
        graph = None
        if cuda_graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            snapshot = [[t.clone() for t in _flat(cache.layer_states[i])] for i in cache.layer_states]
            with torch.cuda.stream(side):
                for _ in range(2):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            for saved, i in zip(snapshot, cache.layer_states):  # the warm-up steps advanced the caches: restore them
                for dst, src in zip(_flat(cache.layer_states[i]), saved):
                    dst.copy_(src)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                logits = step()
            for saved, i in zip(snapshot, cache.layer_states):
                for dst, src in zip(_flat(cache.layer_states[i]), saved):
                    dst.copy_(src)
        out = [input_ids]
        for t in range(max_length - 1):
            tok.copy_(input_ids[:, t:t + 1] if t < plen else nxt)
            if graph is not None:
                graph.replay()
            else:
                logits = step()
            nxt = logits.argmax(-1, keepdim=True)
            if t + 1 >= plen:
                out.append(nxt.clone())
        return torch.cat(out, dim=1)


def _flat(state):
    if isinstance(state, Tensor):
        return [state]
    return [t for s in state for t in _flat(s)]
