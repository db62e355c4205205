"""FSDP / HSDP and activation checkpointing for the vision-language model: encoder layers and decoder blocks are units of
their own (torchtitan/experiments/vlm/infra/parallelize.py:27-187). Tensor / pipeline / context parallel are rejected."""

from __future__ import annotations

import torch.nn as nn

from torchtitan_b200.config import TORCH_DTYPE_MAP
from torchtitan_b200.parallel import fsdp
from torchtitan_b200.parallel.ac import apply_ac
from torchtitan_b200.parallel.fsdp import MixedPrecisionPolicy


def parallelize_vlm(model: nn.Module, *, parallel_dims, training, model_converters, parallelism, compile_config, ac_config,
                    dump_folder: str):
    for name, on in (("tensor", parallel_dims.tp_enabled), ("pipeline", parallel_dims.pp_enabled), ("context", parallel_dims.cp_enabled)):
        if on:
            raise NotImplementedError(f"{name} parallel is not yet supported for the VLM experiment")
    if ac_config.mode != "none":
        apply_ac(model, ac_config, model_compile_enabled=False, base_folder=dump_folder)
    if parallel_dims.fsdp_enabled:
        names = ["dp_replicate", "fsdp"] if parallel_dims.dp_replicate_enabled else ["fsdp"]
        mesh = parallel_dims.get_mesh(names)
        mp = MixedPrecisionPolicy(param_dtype=TORCH_DTYPE_MAP[training.mixed_precision_param],
                                  reduce_dtype=TORCH_DTYPE_MAP[training.mixed_precision_reduce])
        for layer in model.encoder.layers.values():
            fsdp.fully_shard(layer, mesh=mesh, mp_policy=mp)
        for block in model.layers.values():
            fsdp.fully_shard(block, mesh=mesh, mp_policy=mp)
        fsdp.fully_shard(model, mesh=mesh, mp_policy=mp)
    elif parallel_dims.dp_replicate_enabled:
        fsdp.replicate(model, mesh=parallel_dims.get_mesh("dp_replicate"))
    return model
