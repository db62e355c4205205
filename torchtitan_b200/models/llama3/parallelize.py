"""Parallelisation recipe for Llama-3: TP(+SP, loss parallel, async-TP) -> CP -> AC -> data
parallel, the order of torchtitan/models/llama3/parallelize.py:63-172. ``compile.enable`` has
no tracing compiler behind it here and is accepted as a no-op for the model."""

from __future__ import annotations

import torch
import torch.nn as nn

from torchtitan_b200.config import TORCH_DTYPE_MAP
from torchtitan_b200.parallel.ac import apply_ac
from torchtitan_b200.parallel.data_parallel import apply_fsdp, apply_replicate, apply_single_device_units
from torchtitan_b200.tools.logging import logger


def parallelize_llama(model: nn.Module, *, parallel_dims, training, model_converters, parallelism, compile_config,
                      ac_config, dump_folder: str):
    assert training.seq_len % parallel_dims.seq_len_divisor == 0, (
        f"Sequence length {training.seq_len} must be divisible by the product of TP degree "
        f"({parallel_dims.tp}) and 2 * CP degree ({parallel_dims.cp})."
    )
    if parallel_dims.tp_enabled:
        from torchtitan_b200.parallel.tp import apply_tp_to_decoder

        apply_tp_to_decoder(
            model, parallel_dims.get_mesh("tp"), loss_parallel=not parallelism.disable_loss_parallel,
            async_tp=parallelism.enable_async_tensor_parallel, cp_enabled=parallel_dims.cp_enabled,
        )
    if parallel_dims.cp_enabled:
        from torchtitan_b200.parallel.cp import apply_cp_to_attention_module

        apply_cp_to_attention_module(
            [b.attention.inner_attention for b in model.layers.values()], parallel_dims.get_mesh("cp"),
            model.config.layer.attention.attn_backend, rotate_method=parallelism.context_parallel_rotate_method,
            load_balancer=parallelism.context_parallel_load_balancer,
        )
    if ac_config.mode != "none":
        apply_ac(model, ac_config, model_compile_enabled=False, base_folder=dump_folder)
    apply_data_parallel(model, parallel_dims, training, parallelism)
    return model


def apply_data_parallel(model, parallel_dims, training, parallelism):
    param_dtype = TORCH_DTYPE_MAP[training.mixed_precision_param]
    reduce_dtype = TORCH_DTYPE_MAP[training.mixed_precision_reduce]
    if parallel_dims.fsdp_enabled:
        names = ["dp_replicate", "fsdp"] if parallel_dims.dp_replicate_enabled else ["fsdp"]
        apply_fsdp(
            model, parallel_dims.get_mesh(names), param_dtype=param_dtype, reduce_dtype=reduce_dtype,
            pp_enabled=parallel_dims.pp_enabled, cpu_offload=training.enable_cpu_offload,
            reshard_after_forward_policy=parallelism.fsdp_reshard_after_forward, parallelism=parallelism,
            efsdp_mesh=parallel_dims.get_optional_mesh("efsdp") if parallel_dims.ep_enabled else None,
        )
        logger.info("Applied HSDP to the model" if parallel_dims.dp_replicate_enabled else "Applied FSDP to the model")
    elif parallel_dims.dp_replicate_enabled:
        apply_replicate(model, parallel_dims.get_mesh("dp_replicate"), param_dtype=param_dtype, reduce_dtype=reduce_dtype)
    elif torch.cuda.is_available() and training.dtype == "float32" and not parallel_dims.pp_enabled:
        # no data-parallel sharding (one GPU, or tensor parallel only): the same units with a shard world of one keep an
        # fp32 master and a bf16 compute copy, so the bf16 kernels and the flat-shard optimizer still apply
        apply_single_device_units(model, param_dtype=param_dtype, reduce_dtype=reduce_dtype)
        logger.info("Applied single-device mixed-precision units to the model")


# ------------------------------------------------------------------------------------------ building blocks
# the steps a family's parallelize function is made of, under the names the reference's modules give them, for custom
# parallelize functions written against it
from torchtitan_b200.parallel.ac import apply_ac  # noqa: E402,F401
from torchtitan_b200.parallel.data_parallel import apply_fsdp  # noqa: E402,F401
from torchtitan_b200.parallel.ep import apply_moe_ep_tp  # noqa: E402,F401
from torchtitan_b200.parallel.tp import apply_tp_to_decoder as apply_tp  # noqa: E402,F401

apply_non_moe_tp = apply_tp


def apply_compile(model, compile_config=None, **kwargs):
    """No tracing compiler runs in this framework: launch-bound loops are captured in CUDA graphs
    (``experiments/graph_trainer``), the hot operators are kernels of their own."""
    return model


def disable_fsdp_gradient_division(model) -> None:
    """The FSDP units of this framework sum gradients over the data-parallel ranks and never divide: the loss is
    normalised by the global token count. Nothing to switch off."""
    return None
