"""Plan passes of the graph trainer.

Names follow torchtitan/experiments/graph_trainer/passes.py:38-408. Each pass receives the mutable
:class:`StepPlan` and edits it; ``build_plan`` runs the configured passes in order. ``GraphTrainer`` then turns the plan
into settings of the FSDP runtime that the job really runs with: ``parallelism.fsdp_bucket_bytes`` (auto bucketing:
consecutive blocks grouped into one unit), ``fsdp_prefetch_depth`` (units gathered ahead), ``fsdp_reshard_after_forward``,
``fsdp_extra_process_group`` (all-gathers on their own communicator with the c10d transport), per-op activation
checkpointing (``apply_sac``) and CUDA-graph capture of the step (``cudagraph``). ``simple_fsdp.py`` lists the bucket
layouts the two bucketing passes stand for."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

from torchtitan_b200.tools.logging import logger


@dataclass
class StepPlan:
    bucketing: str = "transformer_block"      # "transformer_block" | "auto" | "none"
    bucket_bytes: int = 512 << 20             # target gathered size of an auto bucket
    prefetch_depth: int = 1                   # all-gathers kept in flight ahead of compute
    reshard_after_forward: str = "default"    # default | always | never
    sac_save_ops: set[str] | None = None      # None = leave the eager AC configuration alone
    cudagraph: bool = False
    extra_fsdp_pg: bool = False               # all-gathers on their own process group / stream
    notes: list[str] = field(default_factory=list)


def _default_sac_save_ops() -> set[str]:
    """Ops whose outputs are kept instead of recomputed: GEMMs, attention, and collectives."""
    return {"tt_b200::gemm", "tt_b200::attention_fwd", "aten::mm", "aten::_scaled_dot_product_flash_attention",
            "c10d::reduce_scatter_tensor", "c10d::all_gather_into_tensor", "c10d::all_to_all_single"}


def autobucketing_reordering_pass(plan: StepPlan) -> None:
    plan.bucketing, plan.prefetch_depth = "auto", max(plan.prefetch_depth, 2)


def transformer_block_bucketing_reordering_pass(plan: StepPlan) -> None:
    plan.bucketing, plan.prefetch_depth = "transformer_block", max(plan.prefetch_depth, 1)


def cudagraph_pass(plan: StepPlan) -> None:
    plan.cudagraph = True


def apply_sac_pass(plan: StepPlan) -> None:
    plan.sac_save_ops = _default_sac_save_ops()


def fsdp_reshard_after_fwd_pass(plan: StepPlan) -> None:
    plan.reshard_after_forward = "always"


def reassign_to_pg_pass(plan: StepPlan) -> None:
    plan.extra_fsdp_pg = True


def validate_flex_attn_annotation_pass(plan: StepPlan) -> None:
    plan.notes.append("mask descriptions are plain tensors here; nothing to validate")


def _inductor(name: str) -> Callable[[StepPlan], None]:
    def rejected(plan: StepPlan) -> None:
        raise NotImplementedError(
            f"pass '{name}' lowers the step through the Inductor compiler; this framework runs hand-written sm_100a kernels "
            "and does not use a tracing compiler. Remove it from compile.passes."
        )

    return rejected


AVAILABLE_PASSES: dict[str, Callable[[StepPlan], None]] = {
    "auto_bucketing": autobucketing_reordering_pass,
    "transformer_block_bucketing": transformer_block_bucketing_reordering_pass,
    "cudagraph": cudagraph_pass,
    "apply_sac": apply_sac_pass,
    "fsdp_reshard_after_fwd": fsdp_reshard_after_fwd_pass,
    "reassign_to_pg": reassign_to_pg_pass,
    "validate_flex_attn_annotation": validate_flex_attn_annotation_pass,
    "regional_inductor": _inductor("regional_inductor"),
    "inductor_decomposition": _inductor("inductor_decomposition"),
    "full_inductor_compilation": _inductor("full_inductor_compilation"),
}


def build_plan(passes: list[str], joint_passes: list[str] = ()) -> StepPlan:
    plan = StepPlan()
    names = list(joint_passes) + list(passes)
    if "auto_bucketing" in names and "transformer_block_bucketing" in names:
        raise ValueError("Cannot apply auto_bucketing and transformer_block_bucketing at the same time!")
    if "cudagraph" in names and names[-1] != "cudagraph":
        raise ValueError("cudagraph has to be the last pass to apply")
    for n in names:
        if n not in AVAILABLE_PASSES:
            raise ValueError(f"Unknown pass '{n}'. Available: {sorted(AVAILABLE_PASSES)}")
        AVAILABLE_PASSES[n](plan)
    logger.info(f"graph trainer plan: {plan}")
    return plan
