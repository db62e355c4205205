"""FLUX.1 text-to-image flow-matching model: flavors ``flux-debug``, ``flux-dev``, ``flux-schnell`` (and ``flux-debug-tiny``)
(torchtitan/models/flux/__init__.py)."""

from torchtitan_b200.components.loss import build_mse_loss
from torchtitan_b200.protocols.model_spec import ModelSpec

from .flux_datasets import FluxDataLoader
from .model.state_dict_adapter import FluxStateDictAdapter
from .model.autoencoder import AutoEncoderParams
from .model.model import FluxModel
from .parallelize import parallelize_flux

__all__ = ["FluxModel", "FluxDataLoader", "flux_configs", "parallelize_flux", "model_registry"]

_AE = AutoEncoderParams()

flux_configs = {
    # two double and two single blocks at half the width of flux-dev, full-size autoencoder (the reference's definition)
    "flux-debug": FluxModel.Config(
        in_channels=64, out_channels=64, vec_in_dim=768, context_in_dim=4096, hidden_size=1536, mlp_ratio=4.0, num_heads=12,
        depth=2, depth_single_blocks=2, axes_dim=(16, 56, 56), theta=10_000, qkv_bias=True, autoencoder_params=_AE,
    ),
    # a few million parameters: unit tests and CPU smoke runs
    "flux-debug-tiny": FluxModel.Config(
        in_channels=64, out_channels=64, vec_in_dim=64, context_in_dim=64, hidden_size=256, mlp_ratio=4.0, num_heads=2, depth=2,
        depth_single_blocks=2, axes_dim=(16, 56, 56), theta=10_000, qkv_bias=True,
        autoencoder_params=AutoEncoderParams(resolution=64, ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1),
    ),
    "flux-dev": FluxModel.Config(context_in_dim=4096, autoencoder_params=_AE),
    "flux-schnell": FluxModel.Config(context_in_dim=4096, autoencoder_params=_AE),
}


def model_registry(flavor: str) -> ModelSpec:
    return ModelSpec(name="flux", flavor=flavor, model=flux_configs[flavor], parallelize_fn=parallelize_flux, pipelining_fn=None,
                     build_loss_fn=build_mse_loss, post_optimizer_build_fn=None, state_dict_adapter=FluxStateDictAdapter)
