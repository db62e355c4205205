"""Wrapper that makes a Hugging Face causal LM look like a native decoder.

Parity: torchtitan/experiments/transformers_modeling_backend/model.py:78-700 -- the configuration resolves the
architecture from ``hf_model`` (by ``model_type`` prefix of the id), applies flavor overrides, and the module exposes
``tok_embeddings``, ``layers`` (name -> block mapping), ``norm`` and ``output``; ``forward(tokens)`` returns logits;
``init_weights`` re-runs the architecture's own initialisation; FLOP counting uses the dense formula."""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

import torch
import torch.nn as nn

from torchtitan_b200.models.utils import get_dense_model_nparams_and_flops
from torchtitan_b200.protocols.model import BaseModel
from torchtitan_b200.tools.logging import logger

_ARCH_BY_PREFIX = (("qwen3", "qwen3"), ("qwen2", "qwen2"), ("llama", "llama"), ("mistral", "mistral"), ("gemma", "gemma"),
                   ("phi", "phi3"), ("olmo", "olmo2"))


def _model_type(hf_model: str) -> str:
    name = hf_model.split("/")[-1].lower().replace("-", "").replace("_", "")
    for prefix, mt in _ARCH_BY_PREFIX:
        if name.startswith(prefix) or prefix in name:
            return mt
    return "llama"


class HFTransformerModel(BaseModel):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseModel.Config):
        hf_model: str = "Qwen/Qwen3-4B-Instruct-2507"
        overrides: dict = field(default_factory=dict)
        attn_implementation: str = "sdpa"
        hf_config_path: str = ""
        seq_len: int = 2048

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            hf_model = getattr(trainer_config, "hf_model", "")
            if hf_model:
                self.hf_model = hf_model
            self.seq_len = trainer_config.training.seq_len
            cand = os.path.join(trainer_config.hf_assets_path, "config.json")
            if os.path.exists(cand):
                self.hf_config_path = cand
            par = trainer_config.parallelism
            if par.context_parallel_degree > 1 and par.pipeline_parallel_degree > 1:
                raise NotImplementedError("context parallel and pipeline parallel are not combined for wrapped Hugging Face "
                                          "models")
            if par.pipeline_parallel_degree > 1 and self.hf_config().tie_word_embeddings:
                raise NotImplementedError("pipeline parallel cannot split a model whose output layer shares the embedding "
                                          "weights (tie_word_embeddings)")

        def hf_config(self):
            from transformers import AutoConfig, CONFIG_MAPPING

            if self.hf_config_path:
                with open(self.hf_config_path) as f:
                    raw = json.load(f)
                cfg = CONFIG_MAPPING[raw.get("model_type", _model_type(self.hf_model))](**{k: v for k, v in raw.items() if k != "model_type"})
            else:
                cfg = CONFIG_MAPPING[_model_type(self.hf_model)]()
            for k, v in self.overrides.items():
                setattr(cfg, k, v)
            cfg._attn_implementation = self.attn_implementation
            cfg.use_cache = False
            del AutoConfig
            return cfg

        @property
        def vocab_size(self) -> int:
            return self.hf_config().vocab_size

        @property
        def n_layers(self) -> int:
            return self.hf_config().num_hidden_layers

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int):
            c = self.hf_config()
            head_dim = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
            return get_dense_model_nparams_and_flops(self, model, c.num_attention_heads, 2 * head_dim, seq_len)

    def __init__(self, config: Config):
        super().__init__()
        from transformers import AutoModelForCausalLM

        self.config = config
        self.hf_config = config.hf_config()
        self.model = AutoModelForCausalLM.from_config(self.hf_config, attn_implementation=config.attn_implementation)
        self.model.config.use_cache = False
        logger.info(f"Wrapped Hugging Face architecture {type(self.model).__name__}")

    # ---- native part names -----------------------------------------------------------------------------
    @property
    def _decoder(self):
        return self.model.model if hasattr(self.model, "model") else self.model.transformer

    @property
    def tok_embeddings(self):
        return self._decoder.embed_tokens

    @property
    def layers(self) -> dict[str, nn.Module]:
        return {str(i): m for i, m in enumerate(self._decoder.layers)}

    @property
    def norm(self):
        return self._decoder.norm

    @property
    def output(self):
        return self.model.lm_head

    def forward(self, tokens, attention_masks=None, positions=None):
        if self.__dict__.get("_call_parts_directly"):
            # context parallel: this rank holds a shard of the sequence, so the Hugging Face top-level forward (which
            # builds a causal mask for the local length) is bypassed; the layers call the registered ring attention
            dec = self._decoder
            return _run_parts(dec.embed_tokens, dec.layers, dec.norm, self.model.lm_head, dec.rotary_emb, tokens, positions)
        kw = {}
        if positions is not None:
            kw["position_ids"] = positions.long()
        return self.model(input_ids=tokens, use_cache=False, **kw).logits

    def build_pipeline_stage(self, fqns: list[str]) -> "HFPipelineStage":
        """A pipeline stage holding the named parts (``tok_embeddings``, ``layers.<i>``, ``norm``, ``output``)."""
        return HFPipelineStage(self, fqns)

    def init_weights(self, *args, **kwargs):
        _init_hf_weights(self.model)

    def get_attention_masks(self, input_batch, tokenizer, extra_inputs=None):
        raise TypeError("wrapped Hugging Face models use their own causal masking")


def _init_hf_weights(root: nn.Module, init_fn=None) -> None:
    # buffers such as rotary inverse frequencies are rebuilt by the architecture's own modules
    for m in root.modules():
        if hasattr(m, "inv_freq") and hasattr(m, "rope_init_fn"):
            inv, _ = m.rope_init_fn(m.config, m.inv_freq.device)
            m.inv_freq = inv.to(m.inv_freq.device) if m.inv_freq.device.type != "meta" else inv
            if hasattr(m, "original_inv_freq"):
                m.original_inv_freq = m.inv_freq
    root.apply(init_fn or root._init_weights)


def _run_parts(embed, layers, norm, head, rotary, x, positions):
    """Embedding (if present) -> decoder layers with the architecture's rotary tables -> norm / head (if present). The
    layers get no mask: their attention function runs causal."""
    h = embed(x) if embed is not None else x
    pos = positions.long() if positions is not None else torch.arange(h.shape[1], device=h.device).unsqueeze(0)
    rope = rotary(h, pos)
    for layer in layers:
        out = layer(h, attention_mask=None, position_ids=pos, position_embeddings=rope, use_cache=False)
        h = out[0] if isinstance(out, tuple) else out
    if norm is not None:
        h = norm(h)
    if head is not None:
        h = head(h)
    return h


class _Shell(nn.Module):
    """Container that only gives its children the attribute path they have in the Hugging Face model."""


class HFPipelineStage(nn.Module):
    """Some consecutive parts of a wrapped decoder, run without the Hugging Face top-level ``forward``: embedding (first
    stage), a run of decoder layers with the rotary tables computed by the architecture's own ``rotary_emb``, final norm
    and output head (last stage). Parameters keep the names they have in the whole model
    (``model.model.layers.<i>...``, ``model.lm_head.weight``), so checkpoints do not depend on the pipeline layout.
    Layers are called without an explicit mask: the SDPA attention of the decoder then runs causal, which is what the
    whole model's forward does for full-length sequences; architectures that mix sliding-window layers need their own
    masks and are not covered. Counterpart of torchtitan/experiments/transformers_modeling_backend/pipeline.py:1-415."""

    def __init__(self, whole: "HFTransformerModel", fqns: list[str]):
        super().__init__()
        import copy

        keep = set(fqns)
        self.config, self.hf_config = whole.config, whole.hf_config
        if getattr(self.hf_config, "sliding_window", None) and getattr(self.hf_config, "layer_types", None) and \
                any(t != "full_attention" for t in self.hf_config.layer_types):
            raise NotImplementedError("pipeline stages call decoder layers with plain causal attention; this architecture "
                                      "mixes sliding-window layers")
        src = whole._decoder
        dec = _Shell()
        dec.embed_tokens = copy.deepcopy(src.embed_tokens) if "tok_embeddings" in keep else None
        dec.layers = nn.ModuleDict({str(i): copy.deepcopy(m) for i, m in enumerate(src.layers) if f"layers.{i}" in keep})
        dec.norm = copy.deepcopy(src.norm) if "norm" in keep else None
        dec.rotary_emb = copy.deepcopy(src.rotary_emb)
        top = _Shell()
        top.model = dec
        top.lm_head = copy.deepcopy(whole.model.lm_head) if "output" in keep else None
        self.model = top
        self._init_fn = whole.model._init_weights

    @property
    def tok_embeddings(self):
        return self.model.model.embed_tokens

    @property
    def layers(self) -> dict[str, nn.Module]:
        return dict(self.model.model.layers.items())

    @property
    def norm(self):
        return self.model.model.norm

    @property
    def output(self):
        return self.model.lm_head

    def forward(self, x, attention_masks=None, positions=None):
        dec = self.model.model
        return _run_parts(dec.embed_tokens, dec.layers.values(), dec.norm, self.model.lm_head, dec.rotary_emb, x, positions)

    def init_weights(self, *args, **kwargs):
        _init_hf_weights(self.model, self._init_fn)      # the architecture's initialiser, on this stage's modules

    def get_attention_masks(self, input_batch, tokenizer, extra_inputs=None):
        raise TypeError("wrapped Hugging Face models use their own causal masking")
