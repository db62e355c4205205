"""Cost-model driven automatic sharding.

The reference experiment (torchtitan/experiments/autoparallel: llama3, deepseek_v3 and a ``local_map`` variant) hands the
model to the external ``autoparallel`` package, which searches DTensor placements with a cost model and returns a
parallelised module. That package is not a dependency of this framework: when it is importable the configurations below
delegate to it through ``parallelize_with_autoparallel``; otherwise :func:`auto_plan` provides the built-in planner,
which picks (dp_shard, tp, reshard policy, activation checkpointing) for one NVSwitch node from a memory / bandwidth
model of the B200 (180 GB HBM3e, 7.7 TB/s, NVLink 5).
"""

from .planner import Plan, auto_plan, parallelize_with_autoparallel

__all__ = ["Plan", "auto_plan", "parallelize_with_autoparallel"]
