"""Llama 4: iRoPE decoder with interleaved MoE layers.

Parity: torchtitan/models/llama4/model.py:29-253 -- every ``every_n_layers_nope``-th layer drops
RoPE and attends over the full causal (document) mask, the RoPE layers attend inside fixed blocks
of ``fixed_attn_block_size`` tokens; every ``interleave_moe_layer_step``-th layer is a MoE layer
with a shared expert; the expert hidden size is derived in the original order (2/3 * 4 * dim,
multiplier, divide by top_k + shared, round up). Context parallel is rejected."""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch
import torch.nn as nn

from torchtitan_b200.models.common.attention import AttentionMasks, document_ids
from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.llama3.model import validate_tp_heads
from torchtitan_b200.models.utils import get_moe_model_nparams_and_flops
from torchtitan_b200.tools.logging import logger


def compute_moe_hidden_dim(dim: int, *, multiple_of: int = 256, ffn_dim_multiplier: float | None = None,
                           auto_scale_hidden_dim: bool = True, top_k: int = 1, num_shared_experts: int = 1) -> int:
    hidden = int(2 * (4 * dim) / 3)
    if ffn_dim_multiplier is not None:
        hidden = int(ffn_dim_multiplier * hidden)
    if auto_scale_hidden_dim:
        hidden = int(hidden / (top_k + num_shared_experts))
    return hidden + (-hidden % multiple_of)


class Llama4TransformerBlock(TransformerBlock):
    @dataclass(kw_only=True, slots=True)
    class Config(TransformerBlock.Config):
        depth_init: bool = True
        every_n_layers_nope: int | None = None
        interleave_moe_layer_step: int = 2
        fixed_attn_block_size: int = 8192

    def __init__(self, config: Config, *, layer_id: int, dim: int, n_layers: int):
        super().__init__()
        attn_cfg = config.attention
        if config.every_n_layers_nope is not None:
            if config.every_n_layers_nope <= 1:
                raise ValueError("every_n_layers_nope must be greater than 1")
            if layer_id % config.every_n_layers_nope == 0:
                attn_cfg = dataclasses.replace(attn_cfg, use_rope=False)
        self.attention = attn_cfg.build(dim=dim)
        self.moe_enabled = (layer_id + 1) % config.interleave_moe_layer_step == 0
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
        h = x + self.attention(self.attention_norm(x), freqs_cis, attention_masks, positions)
        ff = self.moe if self.moe_enabled else self.feed_forward
        return h + ff(self.ffn_norm(h))

    def init_weights(self, **kwargs):
        self.attention_norm.init_weights()
        self.ffn_norm.init_weights()
        self.attention.init_weights(self.weight_init_std)
        if self.moe_enabled:
            self.moe.init_weights(init_std=self.weight_init_std, buffer_device=kwargs.get("buffer_device"))
        else:
            self.feed_forward.init_weights(self.weight_init_std)


class Llama4Model(Decoder):
    @dataclass(kw_only=True, slots=True)
    class Config(Decoder.Config):
        dim: int = 4096
        n_layers: int = 32
        vocab_size: int = 202048
        layer: TransformerBlock.Config

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            seq_len = trainer_config.training.seq_len
            par = trainer_config.parallelism
            if seq_len > self.rope.max_seq_len:
                logger.warning(f"Sequence length {seq_len} exceeds original maximum {self.rope.max_seq_len}.")
            self.rope = dataclasses.replace(self.rope, max_seq_len=seq_len)
            assert self.layer.moe is not None
            if par.context_parallel_degree > 1:
                raise NotImplementedError(
                    "Context Parallel is not supported for Llama4 "
                    "(Llama4 requires FlexAttention, which is not supported with CP)."
                )
            self.layer.moe._debug_force_load_balance = trainer_config.debug.moe_force_load_balance
            validate_tp_heads(self.layer.attention, par.tensor_parallel_degree)

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
            n_heads = self.layer.attention.n_heads
            return get_moe_model_nparams_and_flops(self, model, n_heads, 2 * (self.dim // n_heads), seq_len)

    def get_attention_masks(self, input_batch: torch.Tensor, tokenizer, extra_inputs=None):
        """Two mask descriptions keyed by layer kind: RoPE layers add the fixed-block constraint."""
        mask_type = self.config.layer.attention.attn_mask_type
        if mask_type == "causal":
            docs = None
        elif mask_type == "block_causal":
            assert tokenizer.eos_id is not None
            docs = document_ids(input_batch, tokenizer.eos_id)
        else:
            raise ValueError(f"Unknown attention mask type: {mask_type}")
        block = self.config.layer.fixed_attn_block_size
        return {"rope": AttentionMasks(doc_ids=docs, block=block), "nope": AttentionMasks(doc_ids=docs)}
