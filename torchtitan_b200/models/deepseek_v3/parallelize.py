"""DeepSeek-V3 parallelisation: TP over heads for MLA (``wq``/``wq_b``/``wkv_b`` column-wise, ``wo`` row-wise; the
low-rank projections ``wq_a``/``wkv_a`` and their norms stay replicated), MoE EP/TP plan, CP (sdpa only), AC,
MoE-aware FSDP/HSDP. Parity: torchtitan/models/deepseek_v3/parallelize.py:63-341."""

from __future__ import annotations

import torch.nn as nn

from torchtitan_b200.models.llama3.parallelize import apply_data_parallel
from torchtitan_b200.parallel.ac import apply_ac


def parallelize_deepseekv3(model: nn.Module, *, parallel_dims, training, model_converters, parallelism, compile_config,
                           ac_config, dump_folder: str):
    assert training.seq_len % parallel_dims.seq_len_divisor == 0, (
        f"Sequence length {training.seq_len} must be divisible by the product of TP degree "
        f"({parallel_dims.tp}) and 2 * CP degree ({parallel_dims.cp})."
    )
    if parallel_dims.tp_enabled:
        from torchtitan_b200.parallel.tp import apply_tp_to_decoder

        apply_tp_to_decoder(model, parallel_dims.get_mesh("tp"), loss_parallel=not parallelism.disable_loss_parallel,
                            async_tp=parallelism.enable_async_tensor_parallel, cp_enabled=parallel_dims.cp_enabled)
    if parallel_dims.tp_enabled or parallel_dims.ep_enabled:
        from torchtitan_b200.parallel.ep import apply_moe_ep_tp

        apply_moe_ep_tp(model, parallel_dims, parallelism)
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
