"""Llama-3 family model. Parity: torchtitan/models/llama3/model.py:20-134 (depth-scaled init
``0.02 / sqrt(2 (layer_id + 1))`` for output projections, RoPE table resized to the training
sequence length, CP x varlen rejected, TP must divide both head counts)."""

from __future__ import annotations

from dataclasses import dataclass

import torch.nn as nn

from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.utils import get_dense_model_nparams_and_flops


class Llama3TransformerBlock(TransformerBlock):
    """Dense pre-norm block; the two skip connections ride in the output projections' GEMM epilogues."""

    fuse_residual = True

    @dataclass(kw_only=True, slots=True)
    class Config(TransformerBlock.Config):
        depth_init: bool = True

    def __init__(self, config: Config, *, layer_id: int, dim: int, n_layers: int):
        super().__init__()
        self.assemble(config, dim=dim, layer_id=layer_id, n_layers=n_layers, depth_init=config.depth_init)


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
            self.fit_to_job(trainer_config)

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
            heads = self.layer.attention.n_heads
            return get_dense_model_nparams_and_flops(self, model, heads, 2 * (self.dim // heads), seq_len)
