"""Qwen3 flavors: dense 0.6B / 1.7B / 4B / 8B / 14B / 32B (+ debug), MoE ``debugmodel_moe``,
``30B-A3B`` and ``235B-A22B`` (128 experts, top-8 softmax routing with normalised weights, no
shared expert). Table values follow torchtitan/models/qwen3/__init__.py:28-396."""

from torchtitan_b200.components.loss import build_cross_entropy_loss
from torchtitan_b200.components.optimizer import register_moe_load_balancing_hook
from torchtitan_b200.models.common import Embedding, FeedForward, GQAttention, Linear, RMSNorm, RoPE
from torchtitan_b200.models.common.moe import MoE
from torchtitan_b200.parallel.pp import pipeline_llm
from torchtitan_b200.protocols.model_spec import ModelSpec

from .model import Qwen3Model, Qwen3TransformerBlock
from .parallelize import parallelize_qwen3
from .state_dict_adapter import Qwen3StateDictAdapter

__all__ = ["Qwen3Model", "Qwen3TransformerBlock", "qwen3_configs", "model_registry", "parallelize_qwen3"]

_EPS = 1e-6


def _flavor(*, dim, n_layers, n_heads, n_kv_heads, ffn, vocab_size=151936, tie=False, backend="sdpa", mask="causal",
            moe=None, theta=1000000.0, max_seq_len=4096) -> Qwen3Model.Config:
    return Qwen3Model.Config(
        dim=dim, n_layers=n_layers, vocab_size=vocab_size, enable_weight_tying=tie,
        tok_embeddings=Embedding.Config(), norm=RMSNorm.Config(eps=_EPS), output=Linear.Config(),
        layer=Qwen3TransformerBlock.Config(
            attention_norm=RMSNorm.Config(eps=_EPS), ffn_norm=RMSNorm.Config(eps=_EPS),
            feed_forward=FeedForward.Config(hidden_dim=ffn), moe=moe, moe_enabled=moe is not None,
            attention=GQAttention.Config(
                n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=128, q_norm=RMSNorm.Config(eps=_EPS),
                k_norm=RMSNorm.Config(eps=_EPS), attn_backend=backend, attn_mask_type=mask, rope_backend="cos_sin",
            ),
        ),
        rope=RoPE.Config(dim=128, max_seq_len=max_seq_len, theta=theta, backend="cos_sin"),
    )


def _moe(num_experts, hidden):
    return MoE.Config(num_experts=num_experts, num_shared_experts=0, top_k=8, score_func="softmax", route_norm=True,
                      route_scale=1.0, score_before_experts=False, hidden_dim=hidden)


qwen3_configs = {
    "debugmodel": _flavor(dim=256, n_layers=8, n_heads=16, n_kv_heads=8, ffn=3072, vocab_size=2048, tie=True),
    "debugmodel_flex": _flavor(dim=256, n_layers=8, n_heads=16, n_kv_heads=8, ffn=3072, vocab_size=2048, tie=True, backend="flex"),
    "0.6B": _flavor(dim=1024, n_layers=28, n_heads=16, n_kv_heads=8, ffn=3072, tie=True),
    "1.7B": _flavor(dim=2048, n_layers=28, n_heads=16, n_kv_heads=8, ffn=6144, tie=True),
    "4B": _flavor(dim=2560, n_layers=36, n_heads=32, n_kv_heads=8, ffn=9728, tie=True),
    "8B": _flavor(dim=4096, n_layers=36, n_heads=32, n_kv_heads=8, ffn=12288),
    "14B": _flavor(dim=5120, n_layers=40, n_heads=40, n_kv_heads=8, ffn=17408),
    "32B": _flavor(dim=5120, n_layers=64, n_heads=64, n_kv_heads=8, ffn=25600),
    "debugmodel_moe": _flavor(dim=256, n_layers=8, n_heads=16, n_kv_heads=8, ffn=3072, vocab_size=2048, moe=_moe(64, 768)),
    "30B-A3B": _flavor(dim=2048, n_layers=48, n_heads=32, n_kv_heads=4, ffn=6144, moe=_moe(128, 768), max_seq_len=262144),
    "235B-A22B": _flavor(dim=4096, n_layers=94, n_heads=64, n_kv_heads=4, ffn=12288, moe=_moe(128, 1536), theta=5000000.0),
}


def model_registry(flavor: str, *, balance_experts: bool = False) -> ModelSpec:
    """``balance_experts`` registers the auxiliary-loss-free expert-bias update as an optimizer
    pre-hook (the reference leaves it unregistered for Qwen3, so the bias stays zero there)."""
    return ModelSpec(
        name="qwen3",
        flavor=flavor,
        model=qwen3_configs[flavor],
        parallelize_fn=parallelize_qwen3,
        pipelining_fn=pipeline_llm,
        build_loss_fn=build_cross_entropy_loss,
        post_optimizer_build_fn=register_moe_load_balancing_hook if balance_experts else None,
        state_dict_adapter=Qwen3StateDictAdapter,
    )
