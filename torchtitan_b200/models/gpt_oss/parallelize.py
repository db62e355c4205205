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
