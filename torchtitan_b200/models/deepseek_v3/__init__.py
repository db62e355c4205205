"""DeepSeek-V3 flavors ``debugmodel{,_flex_attn}``, ``16B``, ``236B``, ``671B``; values follow
torchtitan/models/deepseek_v3/__init__.py:26-300."""

from torchtitan_b200.components.loss import build_cross_entropy_loss
from torchtitan_b200.components.optimizer import register_moe_load_balancing_hook
from torchtitan_b200.models.common import Embedding, FeedForward, Linear, RMSNorm, RoPE
from torchtitan_b200.models.common.moe import MoE
from torchtitan_b200.parallel.pp import pipeline_llm
from torchtitan_b200.protocols.model_spec import ModelSpec

from .model import Attention, DeepSeekV3Model, DeepSeekV3TransformerBlock
from .parallelize import parallelize_deepseekv3
from .state_dict_adapter import DeepSeekV3StateDictAdapter

__all__ = ["DeepSeekV3Model", "deepseek_v3_configs", "deepseekv3_configs", "model_registry", "parallelize_deepseekv3", "Attention"]


def _rope() -> RoPE.Config:
    return RoPE.Config(dim=64, max_seq_len=4096 * 4, theta=10000.0, backend="complex", scaling="yarn", rope_factor=40.0,
                       beta_fast=32.0, beta_slow=1.0, original_seq_len=4096)


def _flavor(*, dim, n_layers, n_heads, ffn, moe: MoE.Config, vocab_size=102400, n_dense=1, q_lora=0, backend="flex",
            mask="block_causal", mscale=1.0) -> DeepSeekV3Model.Config:
    q = dict(wq=Linear.Config()) if q_lora == 0 else dict(wq_a=Linear.Config(), wq_b=Linear.Config())
    return DeepSeekV3Model.Config(
        vocab_size=vocab_size, dim=dim, n_layers=n_layers,
        tok_embeddings=Embedding.Config(), norm=RMSNorm.Config(), output=Linear.Config(),
        layer=DeepSeekV3TransformerBlock.Config(
            n_dense_layers=n_dense, attention_norm=RMSNorm.Config(), ffn_norm=RMSNorm.Config(), moe=moe,
            attention=Attention.Config(
                q_norm=RMSNorm.Config(), kv_norm=RMSNorm.Config(), n_heads=n_heads, q_lora_rank=q_lora, kv_lora_rank=512,
                qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, mscale=mscale, attn_backend=backend,
                attn_mask_type=mask, **q),
            feed_forward=FeedForward.Config(hidden_dim=ffn),
        ),
        rope=_rope(),
    )


def _moe(**kw) -> MoE.Config:
    base = dict(score_func="softmax", route_norm=False, score_before_experts=False)
    base.update(kw)
    return MoE.Config(**base)


deepseek_v3_configs = {
    "debugmodel": _flavor(dim=256, n_layers=6, n_heads=16, ffn=1024, vocab_size=2048, backend="sdpa", mask="causal", mscale=0.70,
                          moe=_moe(hidden_dim=256, num_experts=8, num_shared_experts=2, top_k=3)),
    "debugmodel_flex_attn": _flavor(dim=256, n_layers=6, n_heads=16, ffn=1024, vocab_size=2048, mscale=0.70,
                                    moe=_moe(hidden_dim=256, num_experts=8, num_shared_experts=2, top_k=3)),
    "16B": _flavor(dim=2048, n_layers=27, n_heads=16, ffn=10944, mscale=0.70,
                   moe=_moe(hidden_dim=1408, num_experts=64, num_shared_experts=2, top_k=6)),
    "236B": _flavor(dim=5120, n_layers=60, n_heads=128, ffn=12288, q_lora=1536,
                    moe=_moe(hidden_dim=1536, num_experts=160, num_shared_experts=2, top_k=6, num_expert_groups=8,
                             num_limited_groups=3, route_scale=16.0)),
    "671B": _flavor(dim=7168, n_layers=61, n_heads=128, ffn=18432, q_lora=1536, vocab_size=129280, n_dense=3,
                    moe=_moe(hidden_dim=2048, num_experts=256, num_shared_experts=1, top_k=8, num_expert_groups=8,
                             num_limited_groups=4, score_func="sigmoid", route_norm=True, route_scale=2.5)),
}
deepseekv3_configs = deepseek_v3_configs      # the spelling of torchtitan/models/deepseek_v3/__init__.py


def model_registry(flavor: str) -> ModelSpec:
    return ModelSpec(
        name="deepseek_v3", flavor=flavor, model=deepseek_v3_configs[flavor], parallelize_fn=parallelize_deepseekv3,
        pipelining_fn=pipeline_llm, build_loss_fn=build_cross_entropy_loss,
        post_optimizer_build_fn=register_moe_load_balancing_hook, state_dict_adapter=DeepSeekV3StateDictAdapter,
    )
