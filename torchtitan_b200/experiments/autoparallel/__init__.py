"""Cost-model driven automatic sharding.

The reference experiment (torchtitan/experiments/autoparallel: llama3, deepseek_v3 and a ``local_map`` variant) hands the
model to the external ``autoparallel`` package, which searches DTensor placements with a cost model and returns a
parallelised module. That package is not a dependency of this framework: when it is importable the configurations below
delegate to it through ``parallelize_with_autoparallel``; otherwise the built-in planner (``planner.py``) searches the
layouts this framework runs -- data-parallel replicate x shard, tensor, pipeline (with schedule), context and expert
parallel, reshard policy, activation checkpointing, on one or several NVSwitch nodes -- with a memory and step-time model
calibrated on this framework's own B200 measurements, and the job configurations below apply its choice.
``python -m torchtitan_b200.experiments.autoparallel.planner --module M --config C --ngpu N`` prints it.
"""

from .planner import ModelShape, Plan, auto_plan, estimate, parallelize_with_autoparallel, search, shape_of

__all__ = ["ModelShape", "Plan", "auto_plan", "estimate", "search", "shape_of", "parallelize_with_autoparallel"]
