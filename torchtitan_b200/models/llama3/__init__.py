"""Llama-3 flavors and ``model_registry``.

Flavor table follows torchtitan/models/llama3/__init__.py:31-263: ``debugmodel`` (dim 256,
6 layers, 16 heads, vocab 2048) and its flex/varlen variants, ``8B`` (32 layers, 32/8 heads,
FFN multiplier 1.3 rounded to 1024 = 14336), ``8B_flex``, ``8B_varlen``, ``70B``, ``405B``;
all with RoPE theta 500000 and Llama-3.1 frequency scaling. ``debugmodel_gqa`` (8 KV heads)
is an addition used by the CPU parity oracle.
"""

from torchtitan_b200.components.loss import build_cross_entropy_loss
from torchtitan_b200.models.common import (
    Embedding, FeedForward, GQAttention, Linear, RMSNorm, RoPE, compute_ffn_hidden_dim,
)
from torchtitan_b200.parallel.pp import pipeline_llm
from torchtitan_b200.protocols.model_spec import ModelSpec

from .model import Llama3Model, Llama3TransformerBlock
from .parallelize import parallelize_llama
from .state_dict_adapter import Llama3StateDictAdapter

__all__ = ["parallelize_llama", "Llama3Model", "Llama3TransformerBlock", "llama3_configs", "model_registry"]


def _flavor(*, dim, n_layers, n_heads, n_kv_heads=None, multiple_of, ffn_mult=None, vocab_size=128256,
            backend="sdpa", mask="causal") -> Llama3Model.Config:
    return Llama3Model.Config(
        dim=dim, n_layers=n_layers, vocab_size=vocab_size,
        tok_embeddings=Embedding.Config(), norm=RMSNorm.Config(), output=Linear.Config(),
        layer=Llama3TransformerBlock.Config(
            attention_norm=RMSNorm.Config(), ffn_norm=RMSNorm.Config(),
            feed_forward=FeedForward.Config(
                hidden_dim=compute_ffn_hidden_dim(dim, multiple_of=multiple_of, ffn_dim_multiplier=ffn_mult)
            ),
            attention=GQAttention.Config(
                n_heads=n_heads, n_kv_heads=n_kv_heads, attn_backend=backend, attn_mask_type=mask,
                rope_backend="complex",
            ),
        ),
        rope=RoPE.Config(dim=dim // n_heads, max_seq_len=131072, theta=500000, backend="complex", scaling="llama"),
    )


_DEBUG = dict(dim=256, n_layers=6, n_heads=16, multiple_of=256, vocab_size=2048)
_8B = dict(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, multiple_of=1024, ffn_mult=1.3)

llama3_configs = {
    "debugmodel": _flavor(**_DEBUG),
    "debugmodel_gqa": _flavor(**_DEBUG, n_kv_heads=8),
    "debugmodel_flex_attn": _flavor(**_DEBUG, backend="flex", mask="block_causal"),
    "debugmodel_varlen_attn": _flavor(**_DEBUG, backend="varlen", mask="block_causal"),
    "8B": _flavor(**_8B),
    "8B_flex": _flavor(**_8B, backend="flex", mask="block_causal"),
    "8B_varlen": _flavor(**_8B, backend="varlen", mask="block_causal"),
    "70B": _flavor(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, multiple_of=4096, ffn_mult=1.3),
    "405B": _flavor(dim=16384, n_layers=126, n_heads=128, n_kv_heads=8, multiple_of=4096, ffn_mult=1.2),
}


def model_registry(flavor: str) -> ModelSpec:
    return ModelSpec(
        name="llama3",
        flavor=flavor,
        model=llama3_configs[flavor],
        parallelize_fn=parallelize_llama,
        pipelining_fn=pipeline_llm,
        build_loss_fn=build_cross_entropy_loss,
        post_optimizer_build_fn=None,
        state_dict_adapter=Llama3StateDictAdapter,
    )
