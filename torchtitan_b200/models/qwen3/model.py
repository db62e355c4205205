"""Qwen3 (dense and MoE). Parity: torchtitan/models/qwen3/model.py:20-191 -- pre-norm block with
per-head QK RMSNorm, half-rotated RoPE (theta 1e6), RMSNorm eps 1e-6, optional weight tying of
embedding and output (not with pipeline parallel), MoE blocks with softmax top-8 routing and no
shared expert; MoE FLOP counting uses active expert parameters only."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from torchtitan_b200.models.common.attention import GQAttention
from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.utils import get_moe_model_nparams_and_flops


class Qwen3TransformerBlock(TransformerBlock):
    @dataclass(kw_only=True, slots=True)
    class Config(TransformerBlock.Config):
        depth_init: bool = True
        moe_enabled: bool = False

    def __init__(self, config: Config, *, layer_id: int, dim: int, n_layers: int):
        super().__init__()
        self.assemble(config, dim=dim, layer_id=layer_id, n_layers=n_layers, moe=config.moe_enabled, depth_init=config.depth_init)


class Qwen3Model(Decoder):
    @dataclass(kw_only=True, slots=True)
    class Config(Decoder.Config):
        dim: int = 1024
        n_layers: int = 28
        vocab_size: int = 151936
        enable_weight_tying: bool = False
        layer: TransformerBlock.Config

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            self.fit_to_job(trainer_config)
            if self.layer.moe is not None:
                self.layer.moe._debug_force_load_balance = trainer_config.debug.moe_force_load_balance
            if self.enable_weight_tying and trainer_config.parallelism.pipeline_parallel_degree > 1:
                raise NotImplementedError("Weight tying is not supported with Pipeline Parallel.")

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
