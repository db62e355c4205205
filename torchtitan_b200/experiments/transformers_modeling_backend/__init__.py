"""Train any Hugging Face ``AutoModelForCausalLM`` architecture with this framework's trainer, FSDP/HSDP runtime and
activation checkpointing. Counterpart of torchtitan/experiments/transformers_modeling_backend (model wrapper exposing
the decoder's ``tok_embeddings / layers / norm / output`` parts under the native names; ``debugmodel`` and ``full``
flavors; ``hf_model`` selects the architecture). FSDP / HSDP, tensor parallel for the usual projection names and pipeline
parallel (stages call the decoder layers directly) apply to wrapped models; context parallel is rejected."""

from torchtitan_b200.components.loss import build_cross_entropy_loss
from torchtitan_b200.parallel.pp import pipeline_llm
from torchtitan_b200.protocols.model_spec import ModelSpec

from .model import HFTransformerModel
from .parallelize import parallelize_hf_transformers

__all__ = ["HFTransformerModel", "model_registry", "parallelize_hf_transformers"]

flavors = {
    # overrides applied on top of the architecture's own configuration
    "debugmodel": dict(hidden_size=256, intermediate_size=768, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=4,
                       head_dim=32, vocab_size=2048, max_position_embeddings=4096, tie_word_embeddings=False),
    "full": {},
}


def model_registry(flavor: str) -> ModelSpec:
    return ModelSpec(
        name="transformers_modeling_backend", flavor=flavor, model=HFTransformerModel.Config(overrides=flavors[flavor]),
        parallelize_fn=parallelize_hf_transformers, pipelining_fn=pipeline_llm, build_loss_fn=build_cross_entropy_loss,
        post_optimizer_build_fn=None, state_dict_adapter=None,
    )
