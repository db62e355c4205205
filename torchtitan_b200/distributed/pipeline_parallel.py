"""Pipeline parallel under the reference's module name (torchtitan/distributed/pipeline_parallel.py)."""

from torchtitan_b200.parallel.pp import (  # noqa: F401
    PipelineSchedule,
    build_actions,
    generate_llm_fqn_per_model_part,
    pipeline_llm,
    pipeline_module_split,
)

__all__ = ["PipelineSchedule", "build_actions", "generate_llm_fqn_per_model_part", "pipeline_llm", "pipeline_module_split"]
