"""Frozen text encoders (T5 encoder and CLIP text model) loaded through ``transformers``; with ``random_init`` a small
randomly initialised model of the same interface is built instead (tests, offline runs).
Parity: torchtitan/models/flux/model/hf_embedder.py."""

from __future__ import annotations

import torch
import torch.nn as nn


class FluxEmbedder(nn.Module):
    def __init__(self, version: str, random_init: bool = False, hidden: int = 64, **hf_kwargs):
        super().__init__()
        self.is_clip = "clip" in version.lower()
        self.output_key = "pooler_output" if self.is_clip else "last_hidden_state"
        if self.is_clip:
            from transformers import CLIPTextConfig, CLIPTextModel

            self.hf_module = (CLIPTextModel(CLIPTextConfig(hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=2,
                                                           num_attention_heads=2, vocab_size=49408, max_position_embeddings=77))
                              if random_init else CLIPTextModel.from_pretrained(version, **hf_kwargs))
        else:
            from transformers import T5Config, T5EncoderModel

            self.hf_module = (T5EncoderModel(T5Config(d_model=hidden, d_ff=2 * hidden, d_kv=hidden // 2, num_layers=2, num_heads=2,
                                                      vocab_size=32128))
                              if random_init else T5EncoderModel.from_pretrained(version, **hf_kwargs))
        self.hf_module = self.hf_module.eval().requires_grad_(False)

    @torch.no_grad()
    def forward(self, batch_tokens: torch.Tensor) -> torch.Tensor:
        out = self.hf_module(input_ids=batch_tokens.to(self.hf_module.device).long(), attention_mask=None, output_hidden_states=False)
        return out[self.output_key]
