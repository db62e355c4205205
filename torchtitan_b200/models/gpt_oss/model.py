"""gpt-oss: attention with learned per-head sink logits, alternating sliding-window / full layers,
MoE in every block. Parity: torchtitan/models/gpt_oss/model.py:33-324. The sink joins only the
softmax denominator, i.e. the plain attention output is multiplied by ``sigmoid(lse - sink)``; even
layers use a 128-token sliding window. Only the ``flex`` backend is accepted, context parallel is
rejected, and there is no pipeline split function."""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from torchtitan_b200.models.common.attention import AttentionMasks, BaseAttention, InnerAttention, document_ids
from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.common.linear import Linear
from torchtitan_b200.models.common.rope import apply_rotary_emb
from torchtitan_b200.models.utils import get_moe_model_nparams_and_flops
from torchtitan_b200.tools.logging import logger


class Attention(BaseAttention):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseAttention.Config):
        n_heads: int = 64
        n_kv_heads: int = 8
        head_dim: int = 64
        linear_bias: bool = False
        attn_backend: str = "flex"
        attn_mask_type: str = "causal"
        sliding_window_size: int = 128

    def __init__(self, config: Config, *, dim: int):
        super().__init__()
        assert config.attn_backend == "flex", "gpt-oss only supports FlexAttention"
        self.head_dim, self.n_heads, self.n_kv_heads = config.head_dim, config.n_heads, config.n_kv_heads
        self.enable_gqa = self.n_heads > self.n_kv_heads
        self.n_rep = self.n_heads // self.n_kv_heads
        self.softmax_scale = 1.0 / math.sqrt(self.head_dim)
        lin = Linear.Config(bias=config.linear_bias)
        self.wq = lin.build(in_features=dim, out_features=config.n_heads * config.head_dim)
        self.wk = lin.build(in_features=dim, out_features=config.n_kv_heads * config.head_dim)
        self.wv = lin.build(in_features=dim, out_features=config.n_kv_heads * config.head_dim)
        self.wo = lin.build(in_features=config.n_heads * config.head_dim, out_features=dim)
        self.sinks = nn.Parameter(torch.empty(config.n_heads))
        self.inner_attention = InnerAttention()

    def init_weights(self, **kwargs):
        init_std = kwargs.get("init_std")
        assert init_std is not None
        nn.init.trunc_normal_(self.sinks, mean=0.0, std=init_std)
        for lin in (self.wq, self.wk, self.wv, self.wo):
            lin.init_weights(init_std=init_std)

    def forward(self, x, freqs_cis, attention_masks, positions=None):
        bsz, seqlen, _ = x.shape
        shape = (bsz, seqlen, -1, self.head_dim)
        q, k, v = self.wq(x).view(shape), self.wk(x).view(shape), self.wv(x).view(shape)
        q, k = apply_rotary_emb(q, k, freqs_cis, positions, "half")
        assert isinstance(attention_masks, AttentionMasks), attention_masks
        sinks = self.sinks.to_local() if hasattr(self.sinks, "to_local") else self.sinks
        out = self.inner_attention(q, k, v, masks=attention_masks, scale=self.softmax_scale, sinks=sinks)
        return self.wo(out.reshape(bsz, seqlen, -1))


class GptOssTransformerBlock(TransformerBlock):
    @dataclass(kw_only=True, slots=True)
    class Config(TransformerBlock.Config):
        pass

    def __init__(self, config: Config, *, layer_id: int, dim: int, n_layers: int):
        super().__init__()
        self.use_sliding_attention = layer_id % 2 == 0
        self.attention = config.attention.build(dim=dim)
        self.attention_norm = config.attention_norm.build(normalized_shape=dim)
        self.ffn_norm = config.ffn_norm.build(normalized_shape=dim)
        assert config.moe is not None
        self.moe = config.moe.build(dim=dim)
        self.moe_enabled = True
        self.weight_init_std = 0.02 / (2 * (layer_id + 1)) ** 0.5
        self.layer_id = layer_id

    def forward(self, x, freqs_cis, attention_masks, positions=None):
        mask = attention_masks.get("sliding_window_mask" if self.use_sliding_attention else "basic_mask")
        assert mask is not None
        x = x + self.attention(self.attention_norm(x), freqs_cis, mask, positions)
        return x + self.moe(self.ffn_norm(x))

    def init_weights(self, **kwargs):
        self.attention_norm.init_weights()
        self.ffn_norm.init_weights()
        self.attention.init_weights(init_std=self.weight_init_std)
        self.moe.init_weights(init_std=self.weight_init_std, buffer_device=kwargs.get("buffer_device"))


class GptOssModel(Decoder):
    @dataclass(kw_only=True, slots=True)
    class Config(Decoder.Config):
        dim: int = 2880
        n_layers: int = 24
        vocab_size: int = 201088
        layer: TransformerBlock.Config

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            seq_len = trainer_config.training.seq_len
            par = trainer_config.parallelism
            if seq_len > self.rope.max_seq_len:
                logger.warning(f"Sequence length {seq_len} exceeds original maximum {self.rope.max_seq_len}.")
            self.rope = dataclasses.replace(self.rope, max_seq_len=seq_len)
            assert self.layer.moe is not None
            if par.context_parallel_degree > 1:
                raise NotImplementedError("CP support for gpt-oss model is still in progress.")
            tp = par.tensor_parallel_degree
            if tp > 1:
                a = self.layer.attention
                if a.n_heads % tp != 0:
                    raise ValueError(f"tensor_parallel_degree ({tp}) must divide n_heads ({a.n_heads}).")
                if a.n_kv_heads % tp != 0:
                    raise ValueError(f"tensor_parallel_degree ({tp}) must divide n_kv_heads ({a.n_kv_heads}).")

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int):
            a = self.layer.attention
            return get_moe_model_nparams_and_flops(self, model, a.n_heads, 2 * a.head_dim, seq_len)

    def get_attention_masks(self, input_batch: torch.Tensor, tokenizer, extra_inputs=None):
        a = self.config.layer.attention
        if a.attn_mask_type == "causal":
            docs = None
        elif a.attn_mask_type == "block_causal":
            assert tokenizer.eos_id is not None
            docs = document_ids(input_batch, tokenizer.eos_id)
        else:
            raise ValueError(f"Unknown attention mask type: {a.attn_mask_type}")
        return {"basic_mask": AttentionMasks(doc_ids=docs),
                "sliding_window_mask": AttentionMasks(doc_ids=docs, window=a.sliding_window_size)}
