"""gpt-oss parallelisation: TP (attention by heads with the sink logits sharded alongside; biases of
column-parallel projections sharded, of row-parallel ones applied once), expert parallel over the
fused ``mlp1/mlp2`` expert tensors, AC, MoE-aware FSDP/HSDP. Pipeline and context parallel are not
offered. Parity: torchtitan/models/gpt_oss/parallelize.py:72-351 and expert_parallel.py:15-71."""

from __future__ import annotations

import torch.nn as nn

from torchtitan_b200.models.llama3.parallelize import apply_data_parallel
from torchtitan_b200.parallel.ac import apply_ac


def parallelize_gptoss(model: nn.Module, *, parallel_dims, training, model_converters, parallelism, compile_config,
                       ac_config, dump_folder: str):
    assert training.seq_len % parallel_dims.seq_len_divisor == 0, (
        f"Sequence length {training.seq_len} must be divisible by the product of TP degree "
        f"({parallel_dims.tp}) and 2 * CP degree ({parallel_dims.cp})."
    )
    if parallel_dims.pp_enabled:
        raise NotImplementedError("Pipeline parallel is not supported for gpt-oss")
    if parallel_dims.tp_enabled:
        from torchtitan_b200.parallel.tp import apply_tp_to_decoder

        apply_tp_to_decoder(model, parallel_dims.get_mesh("tp"), loss_parallel=not parallelism.disable_loss_parallel,
                            async_tp=parallelism.enable_async_tensor_parallel, cp_enabled=False)
    if parallel_dims.tp_enabled or parallel_dims.ep_enabled:
        from torchtitan_b200.parallel.ep import apply_moe_ep_tp

        apply_moe_ep_tp(model, parallel_dims, parallelism)
    if ac_config.mode != "none":
        apply_ac(model, ac_config, model_compile_enabled=False, base_folder=dump_folder)
    apply_data_parallel(model, parallel_dims, training, parallelism)
    return model


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
