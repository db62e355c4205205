"""Qwen3 (dense and MoE). Parity: torchtitan/models/qwen3/model.py:20-191 -- pre-norm block with
per-head QK RMSNorm, half-rotated RoPE (theta 1e6), RMSNorm eps 1e-6, optional weight tying of
embedding and output (not with pipeline parallel), MoE blocks with softmax top-8 routing and no
shared expert; MoE FLOP counting uses active expert parameters only."""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch
import torch.nn as nn

from torchtitan_b200.models.common.attention import GQAttention
from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.llama3.model import validate_tp_heads
from torchtitan_b200.models.utils import get_moe_model_nparams_and_flops
from torchtitan_b200.tools.logging import logger


class Qwen3TransformerBlock(TransformerBlock):
    @dataclass(kw_only=True, slots=True)
    class Config(TransformerBlock.Config):
        depth_init: bool = True
        moe_enabled: bool = False

    def __init__(self, config: Config, *, layer_id: int, dim: int, n_layers: int):
        super().__init__()
        self.attention = config.attention.build(dim=dim)
        self.moe_enabled = config.moe_enabled
        if self.moe_enabled:
            assert config.moe is not None
            self.moe = config.moe.build(dim=dim)
        else:
            assert config.feed_forward is not None
            self.feed_forward = config.feed_forward.build(dim=dim)
        self.attention_norm = config.attention_norm.build(normalized_shape=dim)
        self.ffn_norm = config.ffn_norm.build(normalized_shape=dim)
        depth = (layer_id + 1) if config.depth_init else n_layers
        self.weight_init_std = 0.02 / (2 * depth) ** 0.5

    def forward(self, x, freqs_cis, attention_masks, positions=None):
        x = x + self.attention(self.attention_norm(x), freqs_cis, attention_masks, positions)
        ff = self.moe if self.moe_enabled else self.feed_forward
        return x + ff(self.ffn_norm(x))

    def init_weights(self, **kwargs):
        buffer_device = kwargs.get("buffer_device")
        self.attention_norm.init_weights()
        self.ffn_norm.init_weights()
        self.attention.init_weights(self.weight_init_std)
        if self.moe_enabled:
            self.moe.init_weights(init_std=self.weight_init_std, buffer_device=buffer_device)
        else:
            self.feed_forward.init_weights(self.weight_init_std)


class Qwen3Model(Decoder):
    @dataclass(kw_only=True, slots=True)
    class Config(Decoder.Config):
        dim: int = 1024
        n_layers: int = 28
        vocab_size: int = 151936
        enable_weight_tying: bool = False
        layer: TransformerBlock.Config

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            seq_len = trainer_config.training.seq_len
            par = trainer_config.parallelism
            if seq_len > self.rope.max_seq_len:
                logger.warning(f"Sequence length {seq_len} exceeds original maximum {self.rope.max_seq_len}.")
            self.rope = dataclasses.replace(self.rope, max_seq_len=seq_len)
            if self.layer.moe is not None:
                self.layer.moe._debug_force_load_balance = trainer_config.debug.moe_force_load_balance
            if par.context_parallel_degree > 1 and self.layer.attention.attn_backend == "varlen":
                raise NotImplementedError(
                    "Context Parallel only supports SDPA and FlexAttention. "
                    f"Got attn_backend='{self.layer.attention.attn_backend}'. Varlen attention is not supported with CP."
                )
            if self.enable_weight_tying and par.pipeline_parallel_degree > 1:
                raise NotImplementedError("Weight tying is not supported with Pipeline Parallel.")
            validate_tp_heads(self.layer.attention, par.tensor_parallel_degree)

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
            assert isinstance(self.layer.attention, GQAttention.Config) and self.layer.attention.head_dim is not None
            a = self.layer.attention
            if self.layer.moe is None or not getattr(self.layer, "moe_enabled", False):
                from torchtitan_b200.models.utils import get_dense_model_nparams_and_flops

                return get_dense_model_nparams_and_flops(self, model, a.n_heads, 2 * a.head_dim, seq_len)
            return get_moe_model_nparams_and_flops(self, model, a.n_heads, 2 * a.head_dim, seq_len)

    def __init__(self, config: Config):
        super().__init__(config)
        self.enable_weight_tying = config.enable_weight_tying
        if self.enable_weight_tying:
            self.tok_embeddings.weight = self.output.weight

    def init_weights(self, *, buffer_device: torch.device | None = None, **kwargs):
        if self.enable_weight_tying:
            assert self.tok_embeddings is not None and self.output is not None
            self.tok_embeddings.weight = self.output.weight
        super().init_weights(buffer_device=buffer_device, **kwargs)
