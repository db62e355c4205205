"""DeepSeek-V3: multi-head latent attention (MLA) and dense-then-MoE blocks.

Parity: torchtitan/models/deepseek_v3/model.py:31-334. Queries come from ``wq`` or the low-rank pair
``wq_a -> q_norm -> wq_b``; keys/values from ``wkv_a`` (latent of ``kv_lora_rank`` plus one shared
RoPE key of ``qk_rope_head_dim``) -> ``kv_norm`` -> ``wkv_b``. Each head's query/key is the
concatenation [nope | rope] (128 + 64), values are 128 wide; RoPE uses adjacent-pair rotation. With
a context longer than the original one the softmax scale is multiplied by
``(0.1 * mscale * ln(rope_factor) + 1)^2``. The first ``n_dense_layers`` blocks have a dense FFN, the
rest MoE. ``varlen`` attention is rejected; context parallel needs the sdpa backend."""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from torchtitan_b200.models.common.attention import AttentionMasks, BaseAttention, InnerAttention
from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.common.linear import Linear
from torchtitan_b200.models.common.rmsnorm import RMSNorm
from torchtitan_b200.models.common.rope import apply_rotary_emb_single
from torchtitan_b200.models.utils import get_moe_model_nparams_and_flops
from torchtitan_b200.tools.logging import logger


class Attention(BaseAttention):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseAttention.Config):
        n_heads: int
        wq: Linear.Config | None = None
        wq_a: Linear.Config | None = None
        wq_b: Linear.Config | None = None
        linear_bias: bool = False
        q_lora_rank: int = 0
        kv_lora_rank: int = 512
        q_norm: RMSNorm.Config
        kv_norm: RMSNorm.Config
        qk_nope_head_dim: int = 128
        qk_rope_head_dim: int = 64
        v_head_dim: int = 128
        attn_backend: str = "sdpa"
        attn_mask_type: str = "causal"
        mscale: float = 1.0
        rope_factor: float = 1.0
        rope_max_seq_len: int = 4096
        rope_original_seq_len: int = 4096

    def __init__(self, config: Config, *, dim: int):
        super().__init__()
        if config.attn_backend == "varlen":
            raise ValueError("Varlen attention is not supported with Deepseek V3.")
        self.dim, self.n_heads = dim, config.n_heads
        self.q_lora_rank, self.kv_lora_rank = config.q_lora_rank, config.kv_lora_rank
        self.qk_nope_head_dim, self.qk_rope_head_dim = config.qk_nope_head_dim, config.qk_rope_head_dim
        self.qk_head_dim = config.qk_nope_head_dim + config.qk_rope_head_dim
        self.v_head_dim = config.v_head_dim
        lin = Linear.Config(bias=config.linear_bias)
        if self.q_lora_rank == 0:
            assert config.wq is not None, "wq is required when q_lora_rank == 0"
            assert config.wq.bias == config.linear_bias
            self.wq = config.wq.build(in_features=dim, out_features=self.n_heads * self.qk_head_dim)
        else:
            assert config.wq_a is not None and config.wq_b is not None, "wq_a and wq_b are required when q_lora_rank > 0"
            assert config.wq_a.bias == config.linear_bias and config.wq_b.bias == config.linear_bias
            self.wq_a = config.wq_a.build(in_features=dim, out_features=self.q_lora_rank)
            self.q_norm = config.q_norm.build(normalized_shape=self.q_lora_rank)
            self.wq_b = config.wq_b.build(in_features=self.q_lora_rank, out_features=self.n_heads * self.qk_head_dim)
        self.wkv_a = lin.build(in_features=dim, out_features=self.kv_lora_rank + self.qk_rope_head_dim)
        self.kv_norm = config.kv_norm.build(normalized_shape=self.kv_lora_rank)
        self.wkv_b = lin.build(in_features=self.kv_lora_rank,
                               out_features=self.n_heads * (self.qk_nope_head_dim + self.v_head_dim))
        self.wo = lin.build(in_features=self.n_heads * self.v_head_dim, out_features=dim)
        self.softmax_scale = self.qk_head_dim**-0.5
        if config.rope_max_seq_len > config.rope_original_seq_len:
            m = 0.1 * config.mscale * math.log(config.rope_factor) + 1.0
            self.softmax_scale *= m * m
        self.attn_backend = config.attn_backend
        self.inner_attention = InnerAttention()

    def forward(self, x, freqs_cis, attention_masks, positions=None):
        bsz, seqlen, _ = x.shape
        q = self.wq(x) if self.q_lora_rank == 0 else self.wq_b(self.q_norm(self.wq_a(x)))
        q = q.view(bsz, seqlen, -1, self.qk_head_dim)  # -1: heads are sharded under tensor parallel
        q_nope, q_pe = torch.split(q, [self.qk_nope_head_dim, self.qk_rope_head_dim], dim=-1)
        q_pe = apply_rotary_emb_single(q_pe, freqs_cis, positions, "interleaved")
        q = torch.cat((q_nope, q_pe), dim=-1)
        kv = self.wkv_a(x)
        kv, k_pe = torch.split(kv, [self.kv_lora_rank, self.qk_rope_head_dim], dim=-1)
        k_pe = apply_rotary_emb_single(k_pe.unsqueeze(2), freqs_cis, positions, "interleaved")
        kv = self.wkv_b(self.kv_norm(kv)).view(bsz, seqlen, -1, self.qk_nope_head_dim + self.v_head_dim)
        k_nope, v = torch.split(kv, [self.qk_nope_head_dim, self.v_head_dim], dim=-1)
        k = torch.cat((k_nope, k_pe.expand(-1, -1, k_nope.shape[2], -1)), dim=-1)
        if self.attn_backend == "flex":
            assert isinstance(attention_masks, AttentionMasks)
        else:
            assert attention_masks is None
        out = self.inner_attention(q, k, v, masks=attention_masks, scale=self.softmax_scale)
        return self.wo(out.reshape(bsz, seqlen, -1))

    def init_weights(self, **kwargs) -> None:
        init_std = kwargs.get("init_std")
        assert init_std is not None
        lins = [self.wkv_a, self.wkv_b] + ([self.wq_a, self.wq_b] if self.q_lora_rank > 0 else [self.wq])
        for lin in lins:
            lin.init_weights()
        self.wo.init_weights(init_std=init_std)
        self.kv_norm.init_weights()
        if self.q_lora_rank > 0:
            self.q_norm.init_weights()


class DeepSeekV3TransformerBlock(TransformerBlock):
    @dataclass(kw_only=True, slots=True)
    class Config(TransformerBlock.Config):
        n_dense_layers: int = 1

    def __init__(self, config: Config, *, layer_id: int, dim: int, n_layers: int):
        super().__init__()
        self.attention = config.attention.build(dim=dim)
        self.attention_norm = config.attention_norm.build(normalized_shape=dim)
        self.ffn_norm = config.ffn_norm.build(normalized_shape=dim)
        self.moe_enabled = layer_id >= config.n_dense_layers
        if self.moe_enabled:
            assert config.moe is not None
            self.moe = config.moe.build(dim=dim)
        else:
            assert config.feed_forward is not None
            self.feed_forward = config.feed_forward.build(dim=dim)
        self.weight_init_std = 0.02 / (2 * (layer_id + 1)) ** 0.5
        self.layer_id = layer_id

    def forward(self, x, freqs_cis, attention_masks, positions=None):
        x = x + self.attention(self.attention_norm(x), freqs_cis, attention_masks, positions)
        ff = self.moe if self.moe_enabled else self.feed_forward
        return x + ff(self.ffn_norm(x))

    def init_weights(self, **kwargs):
        self.attention_norm.init_weights()
        self.ffn_norm.init_weights()
        self.attention.init_weights(init_std=self.weight_init_std)
        if self.moe_enabled:
            self.moe.init_weights(init_std=self.weight_init_std, buffer_device=kwargs.get("buffer_device"))
        else:
            self.feed_forward.init_weights(self.weight_init_std)


class DeepSeekV3Model(Decoder):
    @dataclass(kw_only=True, slots=True)
    class Config(Decoder.Config):
        dim: int = 2048
        n_layers: int = 27
        vocab_size: int = 102400
        layer: TransformerBlock.Config

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            seq_len = trainer_config.training.seq_len
            par = trainer_config.parallelism
            if seq_len > self.rope.max_seq_len:
                logger.warning(f"Sequence length {seq_len} exceeds original maximum {self.rope.max_seq_len}.")
            self.rope = dataclasses.replace(self.rope, max_seq_len=seq_len)
            assert isinstance(self.layer.attention, Attention.Config)
            self.layer.attention = dataclasses.replace(
                self.layer.attention, rope_max_seq_len=seq_len, rope_factor=self.rope.rope_factor,
                rope_original_seq_len=self.rope.original_seq_len,
            )
            assert self.layer.moe is not None
            if par.context_parallel_degree > 1 and self.layer.attention.attn_backend != "sdpa":
                raise NotImplementedError(
                    "Context Parallel only supports SDPA attention. "
                    f"Got attn_backend='{self.layer.attention.attn_backend}'. "
                    "FlexAttention and varlen attention are not supported with CP."
                )
            self.layer.moe._debug_force_load_balance = trainer_config.debug.moe_force_load_balance
            tp = par.tensor_parallel_degree
            if tp > 1 and self.layer.attention.n_heads % tp != 0:
                raise ValueError(f"tensor_parallel_degree ({tp}) must divide n_heads ({self.layer.attention.n_heads}).")

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
            a = self.layer.attention
            return get_moe_model_nparams_and_flops(
                self, model, a.n_heads, a.qk_nope_head_dim + a.qk_rope_head_dim + a.v_head_dim, seq_len)
