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
from torchtitan_b200.models.utils import get_moe_model_nparams_and_flops


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
        attention = config.attention
        if config.every_n_layers_nope is not None:
            if config.every_n_layers_nope <= 1:
                raise ValueError("every_n_layers_nope must be greater than 1")
            if layer_id % config.every_n_layers_nope == 0:
                attention = dataclasses.replace(attention, use_rope=False)
        self.assemble(config, dim=dim, layer_id=layer_id, n_layers=n_layers, attention=attention,
                      moe=(layer_id + 1) % config.interleave_moe_layer_step == 0, depth_init=config.depth_init)


class Llama4Model(Decoder):
    @dataclass(kw_only=True, slots=True)
    class Config(Decoder.Config):
        dim: int = 4096
        n_layers: int = 32
        vocab_size: int = 202048
        layer: TransformerBlock.Config

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            assert self.layer.moe is not None
            self.fit_to_job(trainer_config, context_parallel=False)     # needs masks that context parallel does not carry
            self.layer.moe._debug_force_load_balance = trainer_config.debug.moe_force_load_balance

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
