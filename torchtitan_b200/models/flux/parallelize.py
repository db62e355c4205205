"""FSDP / HSDP (one unit per double / single block, one for the embedders + final layer), full or selective activation
checkpointing. Parity: torchtitan/models/flux/parallelize.py."""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from torchtitan_b200.config import TORCH_DTYPE_MAP
from torchtitan_b200.parallel import fsdp
from torchtitan_b200.parallel.fsdp import MixedPrecisionPolicy


def _ckpt(block: nn.Module) -> None:
    inner = block.forward
    block.forward = lambda *a, **k: checkpoint(inner, *a, use_reentrant=False, **k) if torch.is_grad_enabled() else inner(*a, **k)


def parallelize_flux(model: nn.Module, *, parallel_dims, training, model_converters, parallelism, compile_config, ac_config,
                     dump_folder: str):
    if ac_config.mode != "none":
        for b in list(model.double_blocks) + list(model.single_blocks):
            _ckpt(b)
    if parallel_dims.fsdp_enabled:
        names = ["dp_replicate", "fsdp"] if parallel_dims.dp_replicate_enabled else ["fsdp"]
        mesh = parallel_dims.get_mesh(names)
        mp = MixedPrecisionPolicy(param_dtype=TORCH_DTYPE_MAP[training.mixed_precision_param],
                                  reduce_dtype=TORCH_DTYPE_MAP[training.mixed_precision_reduce])
        for b in list(model.double_blocks) + list(model.single_blocks):
            fsdp.fully_shard(b, mesh=mesh, mp_policy=mp)
        fsdp.fully_shard(model, mesh=mesh, mp_policy=mp)
    elif parallel_dims.dp_replicate_enabled:
        fsdp.replicate(model, mesh=parallel_dims.get_mesh("dp_replicate"))
    return model


# the steps of ``parallelize_flux`` under the reference's names, for custom parallelize functions written against it
from torchtitan_b200.parallel.ac import apply_ac  # noqa: E402,F401
from torchtitan_b200.parallel.data_parallel import apply_fsdp  # noqa: E402,F401
