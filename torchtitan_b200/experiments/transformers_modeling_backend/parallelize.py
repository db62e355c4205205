"""Activation checkpointing + FSDP/HSDP for wrapped Hugging Face decoders (one unit per decoder layer, one for
[norm, lm_head], one for the rest). Parity: torchtitan/experiments/transformers_modeling_backend/parallelize.py:41-400,
minus the tensor/context/pipeline plans (rejected in the model configuration)."""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from torchtitan_b200.config import TORCH_DTYPE_MAP
from torchtitan_b200.parallel import fsdp
from torchtitan_b200.parallel.fsdp import MixedPrecisionPolicy
from torchtitan_b200.tools.logging import logger


def _checkpoint_layer(layer: nn.Module) -> None:
    inner = layer.forward

    def forward(*args, **kwargs):
        if not torch.is_grad_enabled():
            return inner(*args, **kwargs)
        return checkpoint(inner, *args, use_reentrant=False, **kwargs)

    layer.forward = forward


def parallelize_hf_transformers(model: nn.Module, *, parallel_dims, training, model_converters, parallelism, compile_config,
                                ac_config, dump_folder: str):
    layers = list(model.layers.values())
    if ac_config.mode == "full":
        for layer in layers:
            _checkpoint_layer(layer)
    elif ac_config.mode == "selective":
        every = int(ac_config.selective_ac_option) if str(ac_config.selective_ac_option).isdigit() else 1
        for i, layer in enumerate(layers):
            if every and (i + 1) % every == 0:
                _checkpoint_layer(layer)
    if parallel_dims.fsdp_enabled or parallel_dims.dp_replicate_enabled:
        mesh = parallel_dims.get_mesh(["dp_replicate", "fsdp"] if parallel_dims.dp_replicate_enabled and parallel_dims.fsdp_enabled
                                      else ("fsdp" if parallel_dims.fsdp_enabled else "dp_replicate"))
        mp = MixedPrecisionPolicy(param_dtype=TORCH_DTYPE_MAP[training.mixed_precision_param],
                                  reduce_dtype=TORCH_DTYPE_MAP[training.mixed_precision_reduce])
        if parallel_dims.fsdp_enabled:
            for layer in layers:
                fsdp.fully_shard(layer, mesh=mesh, mp_policy=mp)
            if not getattr(model.hf_config, "tie_word_embeddings", False):
                fsdp.fully_shard([model.norm, model.output], mesh=mesh, mp_policy=mp)
            fsdp.fully_shard(model, mesh=mesh, mp_policy=mp)
            logger.info("Applied FSDP to the wrapped Hugging Face model")
        else:
            fsdp.replicate(model, mesh=mesh, mp_policy=mp)
            logger.info("Applied DDP to the wrapped Hugging Face model")
    return model
