"""Llama 4 flavors ``debugmodel``, ``17bx16e`` (Scout) and ``17bx128e`` (Maverick); table values
follow torchtitan/models/llama4/__init__.py:31-163."""

from torchtitan_b200.components.loss import build_cross_entropy_loss
from torchtitan_b200.components.optimizer import register_moe_load_balancing_hook
from torchtitan_b200.models.common import Embedding, FeedForward, GQAttention, Linear, RMSNorm, RoPE, compute_ffn_hidden_dim
from torchtitan_b200.models.common.moe import MoE
from torchtitan_b200.parallel.pp import pipeline_llm
from torchtitan_b200.protocols.model_spec import ModelSpec

from .model import Llama4Model, Llama4TransformerBlock, compute_moe_hidden_dim
from .parallelize import parallelize_llama
from .state_dict_adapter import Llama4StateDictAdapter  # noqa: F401

__all__ = ["Llama4Model", "llama4_configs", "model_registry", "parallelize_llama", "compute_moe_hidden_dim"]


def _big(num_experts: int, *, moe_step: int, max_seq_len: int, scaled: bool) -> Llama4Model.Config:
    rope = dict(scaling="llama", scaling_factor=16.0, high_freq_factor=1.0) if scaled else dict(scaling="none")
    return Llama4Model.Config(
        dim=5120, n_layers=48, tok_embeddings=Embedding.Config(), norm=RMSNorm.Config(), output=Linear.Config(),
        layer=Llama4TransformerBlock.Config(
            every_n_layers_nope=4, interleave_moe_layer_step=moe_step,
            attention_norm=RMSNorm.Config(), ffn_norm=RMSNorm.Config(),
            moe=MoE.Config(num_experts=num_experts, hidden_dim=compute_moe_hidden_dim(
                5120, multiple_of=2048, ffn_dim_multiplier=1.2, top_k=1, num_shared_experts=1)),
            feed_forward=FeedForward.Config(hidden_dim=compute_ffn_hidden_dim(5120, multiple_of=2048, ffn_dim_multiplier=1.2)),
            attention=GQAttention.Config(n_heads=40, n_kv_heads=8, attn_backend="flex", attn_mask_type="block_causal",
                                         rope_backend="complex"),
        ),
        rope=RoPE.Config(dim=5120 // 40, max_seq_len=max_seq_len, theta=500000, backend="complex", **rope),
    )


llama4_configs = {
    "debugmodel": Llama4Model.Config(
        dim=256, n_layers=6, vocab_size=2048, tok_embeddings=Embedding.Config(), norm=RMSNorm.Config(), output=Linear.Config(),
        layer=Llama4TransformerBlock.Config(
            every_n_layers_nope=4, fixed_attn_block_size=256,
            attention_norm=RMSNorm.Config(), ffn_norm=RMSNorm.Config(),
            feed_forward=FeedForward.Config(hidden_dim=compute_ffn_hidden_dim(256, multiple_of=256)),
            attention=GQAttention.Config(n_heads=16, attn_backend="flex", attn_mask_type="block_causal", rope_backend="complex"),
            moe=MoE.Config(hidden_dim=compute_moe_hidden_dim(256)),
        ),
        rope=RoPE.Config(dim=256 // 16, max_seq_len=1048576, theta=500000, backend="complex", scaling="llama",
                         scaling_factor=16.0, high_freq_factor=1.0),
    ),
    "17bx16e": _big(16, moe_step=1, max_seq_len=10485760, scaled=True),
    "17bx128e": _big(128, moe_step=2, max_seq_len=1048576, scaled=False),
}


def model_registry(flavor: str) -> ModelSpec:
    return ModelSpec(
        name="llama4", flavor=flavor, model=llama4_configs[flavor], parallelize_fn=parallelize_llama,
        pipelining_fn=pipeline_llm, build_loss_fn=build_cross_entropy_loss,
        post_optimizer_build_fn=register_moe_load_balancing_hook, state_dict_adapter=Llama4StateDictAdapter,
    )
