"""Pipeline parallel under the reference's module name (torchtitan/distributed/pipeline_parallel.py)."""

from torchtitan_b200.parallel.pp import (  # noqa: F401
    PipelineSchedule,
    build_actions,
    generate_llm_fqn_per_model_part,
    pipeline_llm,
    pipeline_module_split,
)

__all__ = ["PipelineSchedule", "build_actions", "build_pipeline_schedule", "generate_llm_fqn_per_model_part", "pipeline_llm",
           "pipeline_module_split"]


def build_pipeline_schedule(*args, **kwargs):
    """The reference assembles a ``torch.distributed.pipelining`` schedule object from stages here
    (pipeline_parallel.py:134-238); this framework's runtime is built by :func:`pipeline_llm`, which cuts the model,
    parallelises the parts and returns the :class:`PipelineSchedule` in one call."""
    raise NotImplementedError("use torchtitan_b200.parallel.pp.pipeline_llm, which returns the schedule with its stages")
