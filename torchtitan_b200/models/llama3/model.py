"""Llama-3 family model. Parity: torchtitan/models/llama3/model.py:20-134 (depth-scaled init
``0.02 / sqrt(2 (layer_id + 1))`` for output projections, RoPE table resized to the training
sequence length, CP x varlen rejected, TP must divide both head counts)."""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch.nn as nn

from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.common.linear import with_residual
from torchtitan_b200.models.utils import get_dense_model_nparams_and_flops
from torchtitan_b200.tools.logging import logger


class Llama3TransformerBlock(TransformerBlock):
    @dataclass(kw_only=True, slots=True)
    class Config(TransformerBlock.Config):
        depth_init: bool = True

    def __init__(self, config: Config, *, layer_id: int, dim: int, n_layers: int):
        super().__init__()
        assert config.feed_forward is not None
        self.attention = config.attention.build(dim=dim)
        self.feed_forward = config.feed_forward.build(dim=dim)
        self.attention_norm = config.attention_norm.build(normalized_shape=dim)
        self.ffn_norm = config.ffn_norm.build(normalized_shape=dim)
        depth = (layer_id + 1) if config.depth_init else n_layers
        self.weight_init_std = 0.02 / (2 * depth) ** 0.5

    def forward(self, x, freqs_cis, attention_masks, positions=None):
        # the skip connections are handed to the output projections, which add them in their GEMM epilogues
        h = with_residual(self.attention, x, self.attention_norm(x), freqs_cis, attention_masks, positions)
        return with_residual(self.feed_forward, h, self.ffn_norm(h))

    def init_weights(self, **kwargs):
        self.attention_norm.init_weights()
        self.ffn_norm.init_weights()
        self.attention.init_weights(self.weight_init_std)
        self.feed_forward.init_weights(self.weight_init_std)


def validate_tp_heads(attn_cfg, tp: int) -> None:
    if tp <= 1:
        return
    n_heads = attn_cfg.n_heads
    n_kv = getattr(attn_cfg, "n_kv_heads", None) or n_heads
    if n_heads % tp != 0:
        raise ValueError(f"tensor_parallel_degree ({tp}) must divide n_heads ({n_heads}).")
    if n_kv % tp != 0:
        raise ValueError(f"tensor_parallel_degree ({tp}) must divide n_kv_heads ({n_kv}).")


class Llama3Model(Decoder):
    @dataclass(kw_only=True, slots=True)
    class Config(Decoder.Config):
        dim: int = 4096
        n_layers: int = 32
        vocab_size: int = 128256
        layer: TransformerBlock.Config

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            seq_len = trainer_config.training.seq_len
            par = trainer_config.parallelism
            if seq_len > self.rope.max_seq_len:
                logger.warning(f"Sequence length {seq_len} exceeds original maximum {self.rope.max_seq_len}.")
            self.rope = dataclasses.replace(self.rope, max_seq_len=seq_len)
            if par.context_parallel_degree > 1 and self.layer.attention.attn_backend == "varlen":
                raise NotImplementedError(
                    "Context Parallel only supports SDPA and FlexAttention. "
                    f"Got attn_backend='{self.layer.attention.attn_backend}'. "
                    "Varlen attention is not supported with CP."
                )
            validate_tp_heads(self.layer.attention, par.tensor_parallel_degree)

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
            heads = self.layer.attention.n_heads
            return get_dense_model_nparams_and_flops(self, model, heads, 2 * (self.dim // heads), seq_len)
