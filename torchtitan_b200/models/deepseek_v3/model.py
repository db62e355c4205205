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
        c = config
        self.dim, self.n_heads = dim, c.n_heads
        self.q_lora_rank, self.kv_lora_rank = c.q_lora_rank, c.kv_lora_rank
        self.qk_nope_head_dim, self.qk_rope_head_dim, self.v_head_dim = c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim
        self.qk_head_dim = c.qk_nope_head_dim + c.qk_rope_head_dim
        plain = Linear.Config(bias=c.linear_bias)
        # projections as a table: name -> (config, in, out); the query side is either one matrix or a low-rank pair
        q_out = self.n_heads * self.qk_head_dim
        if self.q_lora_rank == 0:
            table = {"wq": (c.wq, dim, q_out)}
        else:
            table = {"wq_a": (c.wq_a, dim, self.q_lora_rank), "wq_b": (c.wq_b, self.q_lora_rank, q_out)}
        for name, (cfg, _, _) in table.items():
            if cfg is None:
                raise AssertionError(f"{name} is required when q_lora_rank {'== 0' if name == 'wq' else '> 0'}")
            assert cfg.bias == c.linear_bias, f"{name}.bias must equal linear_bias"
        table.update({
            "wkv_a": (plain, dim, self.kv_lora_rank + self.qk_rope_head_dim),
            "wkv_b": (plain, self.kv_lora_rank, self.n_heads * (self.qk_nope_head_dim + self.v_head_dim)),
            "wo": (plain, self.n_heads * self.v_head_dim, dim),
        })
        for name, (cfg, fin, fout) in table.items():
            setattr(self, name, cfg.build(in_features=fin, out_features=fout))
        if self.q_lora_rank > 0:
            self.q_norm = c.q_norm.build(normalized_shape=self.q_lora_rank)
        self.kv_norm = c.kv_norm.build(normalized_shape=self.kv_lora_rank)
        self.softmax_scale = self._scale(c)
        self.attn_backend = c.attn_backend
        self.inner_attention = InnerAttention()

    def _scale(self, c) -> float:
        """1 / sqrt(query width), times the YaRN attention factor squared once the context exceeds the original one."""
        scale = self.qk_head_dim**-0.5
        if c.rope_max_seq_len > c.rope_original_seq_len:
            scale *= (0.1 * c.mscale * math.log(c.rope_factor) + 1.0) ** 2
        return scale

    def _queries(self, x, freqs_cis, positions):
        """[B, S, heads, nope + rope]: the rope slice of every head is rotated (adjacent pairs), the rest passes through."""
        q = self.wq(x) if self.q_lora_rank == 0 else self.wq_b(self.q_norm(self.wq_a(x)))
        q = q.unflatten(-1, (-1, self.qk_head_dim))              # heads may be a tensor-parallel shard
        rot = apply_rotary_emb_single(q[..., self.qk_nope_head_dim:], freqs_cis, positions, "interleaved")
        return torch.cat((q[..., : self.qk_nope_head_dim], rot), dim=-1)

    def _keys_values(self, x, freqs_cis, positions):
        """Latent -> per-head keys [nope | shared rotated rope key] and values."""
        latent, k_rope = self.wkv_a(x).split([self.kv_lora_rank, self.qk_rope_head_dim], dim=-1)
        k_rope = apply_rotary_emb_single(k_rope.unsqueeze(2), freqs_cis, positions, "interleaved")   # one key for all heads
        kv = self.wkv_b(self.kv_norm(latent)).unflatten(-1, (-1, self.qk_nope_head_dim + self.v_head_dim))
        k_nope, v = kv.split([self.qk_nope_head_dim, self.v_head_dim], dim=-1)
        return torch.cat((k_nope, k_rope.expand(-1, -1, k_nope.shape[2], -1)), dim=-1), v

    def forward(self, x, freqs_cis, attention_masks, positions=None):
        if self.attn_backend == "flex":
            assert isinstance(attention_masks, AttentionMasks)
        else:
            assert attention_masks is None
        q = self._queries(x, freqs_cis, positions)
        k, v = self._keys_values(x, freqs_cis, positions)
        # 192-wide queries / keys and 128-wide values: the attention kernels have an instantiation for this pair
        out = self.inner_attention(q, k, v.contiguous(), masks=attention_masks, scale=self.softmax_scale)
        return self.wo(out.flatten(2))

    def init_weights(self, **kwargs) -> None:
        init_std = kwargs.get("init_std")
        assert init_std is not None
        for name, mod in self.named_children():
            if name == "wo":
                mod.init_weights(init_std=init_std)
            elif name != "inner_attention":
                mod.init_weights()


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
