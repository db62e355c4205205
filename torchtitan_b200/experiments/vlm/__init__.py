"""Vision-language model experiment: Llama 3 decoder + SigLIP2-style native-resolution vision encoder.

Parity: torchtitan/experiments/vlm (model/model.py, model/siglip2.py, datasets/*, infra/parallelize.py): images are
cut into patches at their native aspect ratio, each image becomes a row of a padded ``[N, L, patch_dim]`` tensor with
per-patch grid coordinates, the encoder output is projected and written into the positions of ``<|image|>`` placeholder
tokens of the text sequence; samples are packed into fixed-length sequences."""

from torchtitan_b200.components.loss import build_cross_entropy_loss
from torchtitan_b200.models.llama3 import llama3_configs
from torchtitan_b200.protocols.model_spec import ModelSpec

from .model import Llama3Siglip2Transformer, Siglip2Config, SpecialTokens
from .parallelize import parallelize_vlm

__all__ = ["Llama3Siglip2Transformer", "Siglip2Config", "SpecialTokens", "model_registry", "llama3_siglip2_configs",
           "HuggingFaceMultiModalDataLoader"]


def __getattr__(name):          # the loader pulls in the dataset stack: imported on first use
    if name == "HuggingFaceMultiModalDataLoader":
        from .datasets import MMDataLoader

        return MMDataLoader
    raise AttributeError(name)


def _from_llama(flavor: str, encoder: Siglip2Config) -> Llama3Siglip2Transformer.Config:
    import dataclasses

    base = llama3_configs[flavor]
    fields = {f.name: getattr(base, f.name) for f in dataclasses.fields(base)}
    return Llama3Siglip2Transformer.Config(encoder=encoder, **fields)


llama3_siglip2_configs = {
    "debugmodel": _from_llama("debugmodel_flex_attn", Siglip2Config(dim=128, ffn_dim=256, n_layers=4, n_heads=2)),
    "8B": _from_llama("8B_flex", Siglip2Config()) if "8B_flex" in llama3_configs else _from_llama("8B", Siglip2Config()),
}


def model_registry(flavor: str) -> ModelSpec:
    return ModelSpec(
        name="vlm", flavor=flavor, model=llama3_siglip2_configs[flavor], parallelize_fn=parallelize_vlm, pipelining_fn=None,
        build_loss_fn=build_cross_entropy_loss, post_optimizer_build_fn=None, state_dict_adapter=None,
    )
