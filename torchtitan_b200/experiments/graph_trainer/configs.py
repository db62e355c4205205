"""Configuration of the graph trainer (fields as in torchtitan/experiments/graph_trainer/configs.py:16-70)."""

from collections.abc import Callable
from dataclasses import dataclass, field, fields
from typing import Literal

from torchtitan_b200.config import CompileConfig
from torchtitan_b200.protocols.model_spec import ModelSpec
from torchtitan_b200.trainer import Trainer


@dataclass(kw_only=True, slots=True)
class GraphTrainerCompileConfig(CompileConfig):
    mode: Literal["jit", "aot"] | None = "aot"
    """Kept for compatibility: both modes build the same run-time plan here."""
    backend: str = "aot_eager"
    passes: list[str] = field(default_factory=list)
    """Plan passes, applied in order (see ``passes.AVAILABLE_PASSES``)."""
    joint_passes: list[str] = field(default_factory=list)
    """Passes that act on forward and backward together (``apply_sac``, ``fsdp_reshard_after_fwd``...)."""


@dataclass(kw_only=True, slots=True)
class GraphTrainerConfig(Trainer.Config):
    compile: GraphTrainerCompileConfig = field(default_factory=GraphTrainerCompileConfig)


def to_graph_trainer_config(base_config: Trainer.Config, model_registry: Callable[[str], ModelSpec]):
    """Copy a base trainer configuration, swap in the graph-trainer model spec and reset ``compile``."""
    from .trainer import GraphTrainer

    d = {f.name: getattr(base_config, f.name) for f in fields(base_config)}
    d["model_spec"] = model_registry(base_config.model_spec.flavor)
    d.pop("compile")
    return GraphTrainer.Config(**d)
