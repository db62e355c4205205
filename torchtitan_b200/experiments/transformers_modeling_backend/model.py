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
            for name, deg in (("context", par.context_parallel_degree), ("pipeline", par.pipeline_parallel_degree)):
                if deg > 1:
                    raise NotImplementedError(f"{name} parallel is not available for wrapped Hugging Face models; "
                                              "use FSDP / HSDP and tensor parallel")

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
        kw = {}
        if positions is not None:
            kw["position_ids"] = positions.long()
        return self.model(input_ids=tokens, use_cache=False, **kw).logits

    def init_weights(self, *args, **kwargs):
        # buffers such as rotary inverse frequencies are rebuilt by the architecture's own modules
        for m in self.model.modules():
            if hasattr(m, "inv_freq") and hasattr(m, "rope_init_fn"):
                inv, _ = m.rope_init_fn(m.config, m.inv_freq.device)
                m.inv_freq = inv.to(m.inv_freq.device) if m.inv_freq.device.type != "meta" else inv
                if hasattr(m, "original_inv_freq"):
                    m.original_inv_freq = m.inv_freq
        self.model.apply(self.model._init_weights)

    def get_attention_masks(self, input_batch, tokenizer, extra_inputs=None):
        raise TypeError("wrapped Hugging Face models use their own causal masking")
