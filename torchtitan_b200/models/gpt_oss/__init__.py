"""gpt-oss flavors ``debugmodel``, ``20b`` (32 experts) and ``120b`` (128 experts, 36 layers); values follow
torchtitan/models/gpt_oss/__init__.py:23-140. No pipeline split function is registered."""

from torchtitan_b200.components.loss import build_cross_entropy_loss
from torchtitan_b200.components.optimizer import register_moe_load_balancing_hook
from torchtitan_b200.models.common import Embedding, Linear, RMSNorm, RoPE
from torchtitan_b200.protocols.model_spec import ModelSpec

from .model import Attention, GptOssModel, GptOssTransformerBlock
from .moe import GptOssMoE
from .parallelize import parallelize_gptoss
from .state_dict_adapter import GptOssStateDictAdapter

__all__ = ["parallelize_gptoss", "GptOssModel", "gptoss_configs", "model_registry"]


def _flavor(num_experts: int, **top) -> GptOssModel.Config:
    return GptOssModel.Config(
        tok_embeddings=Embedding.Config(), norm=RMSNorm.Config(), output=Linear.Config(),
        layer=GptOssTransformerBlock.Config(
            attention_norm=RMSNorm.Config(), ffn_norm=RMSNorm.Config(),
            moe=GptOssMoE.Config(hidden_dim=2880, num_experts=num_experts, num_shared_experts=0, score_func="softmax",
                                 route_norm=True, route_scale=1.0, gate_bias=True, score_before_experts=False, top_k=4,
                                 use_grouped_mm=True, load_balance_coeff=1e-3),
            attention=Attention.Config(linear_bias=True),
        ),
        rope=RoPE.Config(dim=64, max_seq_len=131072, theta=150000.0, backend="cos_sin", scaling="yarn", rope_factor=32,
                         beta_slow=32.0, beta_fast=1.0, original_seq_len=4096),
        **top,
    )


gptoss_configs = {
    "debugmodel": _flavor(8, vocab_size=2048, dim=256, n_layers=4),
    "20b": _flavor(32, n_layers=24),
    "120b": _flavor(128, n_layers=36),
}


def model_registry(flavor: str) -> ModelSpec:
    return ModelSpec(
        name="gpt_oss", flavor=flavor, model=gptoss_configs[flavor], parallelize_fn=parallelize_gptoss, pipelining_fn=None,
        build_loss_fn=build_cross_entropy_loss, post_optimizer_build_fn=register_moe_load_balancing_hook,
        state_dict_adapter=GptOssStateDictAdapter,
    )
