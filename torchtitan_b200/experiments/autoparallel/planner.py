"""A small analytic planner for one node and the bridge to the external ``autoparallel`` package."""

from __future__ import annotations

from dataclasses import dataclass

HBM_BYTES = 180e9
HBM_BW = 6.5e12          # measured copy bandwidth, bytes/s
NVLINK_BW = 770e9        # measured peer copy bandwidth per direction, bytes/s
BF16_FLOPS = 1.4e15      # sustained dense bf16


@dataclass
class Plan:
    dp_shard: int
    tp: int
    reshard_after_forward: str
    ac_mode: str
    est_step_s: float
    est_mem_bytes: float

    def to_overrides(self) -> list[str]:
        return [f"--parallelism.data_parallel_shard_degree={self.dp_shard}", f"--parallelism.tensor_parallel_degree={self.tp}",
                f"--parallelism.fsdp_reshard_after_forward={self.reshard_after_forward}", f"--activation_checkpoint.mode={self.ac_mode}"]


def _estimate(nparams: float, flops_per_token: float, tokens_per_gpu: int, act_bytes_per_token_layer: float, n_layers: int,
              dp: int, tp: int, reshard: str, ac: str) -> tuple[float, float]:
    # memory: fp32 master + 2 Adam moments + fp32 grad shard (16 B / param / (dp*tp)), bf16 gathered copy or one unit
    mem = 16.0 * nparams / (dp * tp)
    mem += 2.0 * nparams / tp if reshard == "never" else 2.0 * nparams / tp / max(n_layers, 1) * 2
    act = act_bytes_per_token_layer * tokens_per_gpu * n_layers / tp
    mem += act * {"none": 1.0, "selective": 0.45, "full": 0.08}[ac]
    # time: compute (+ recompute), FSDP gathers that cannot hide, TP collectives on the critical path
    compute = flops_per_token * tokens_per_gpu / tp / BF16_FLOPS * {"none": 1.0, "selective": 1.08, "full": 1.33}[ac]
    gathers = (2 if reshard == "never" else 3) * 2.0 * nparams / tp * (dp - 1) / dp / NVLINK_BW if dp > 1 else 0.0
    tp_comm = 0.0 if tp == 1 else 8.0 * n_layers * tokens_per_gpu * (nparams / n_layers / 12) ** 0.5 * 2 * (tp - 1) / tp / NVLINK_BW
    return compute + max(0.0, gathers - 0.7 * compute) + tp_comm, mem


def auto_plan(nparams: int, flops_per_token: float, n_layers: int, dim: int, seq_len: int, local_batch: int,
              world_size: int) -> Plan:
    """Exhaustive search over the (small) plan space of one node; cheapest estimated step that fits in memory."""
    tokens = seq_len * local_batch
    act = 34.0 * dim   # bytes per token per layer kept for backward without checkpointing (bf16 activations of a block)
    best = None
    for tp in (t for t in (1, 2, 4, 8) if world_size % t == 0):
        dp = world_size // tp
        for reshard in ("never", "always"):
            for ac in ("none", "selective", "full"):
                t, m = _estimate(nparams, flops_per_token, tokens, act, n_layers, dp, tp, reshard, ac)
                if m > 0.92 * HBM_BYTES:
                    continue
                # objective: time per globally processed token (a TP group shares one local batch)
                if best is None or t / dp < best.est_step_s / best.dp_shard:
                    best = Plan(dp, tp, reshard, ac, t, m)
    if best is None:
        raise RuntimeError("no plan fits in memory on this node; add pipeline parallel or more nodes")
    return best


def parallelize_with_autoparallel(model, mesh, input_fn, **kwargs):
    """Delegate to the external package when it is installed (same call the reference experiment makes)."""
    try:
        from autoparallel.api import AutoParallel  # type: ignore
    except ImportError as e:
        raise ImportError("the 'autoparallel' package is not installed; use experiments.autoparallel.auto_plan "
                          "for the built-in single-node planner") from e
    with AutoParallel(model, input_fn, mesh, **kwargs) as autop:
        autop.add_parameter_memory_constraint(low=None, high=None)
        placement = autop.optimize_placement()
        return autop.apply_placement(placement)
