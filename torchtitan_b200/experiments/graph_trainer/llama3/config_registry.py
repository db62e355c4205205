"""Graph-trainer job configurations for Llama 3 (names follow
torchtitan/experiments/graph_trainer/llama3/config_registry.py)."""

from torchtitan_b200.experiments.graph_trainer.configs import GraphTrainerCompileConfig, to_graph_trainer_config
from torchtitan_b200.models.llama3 import config_registry as base

from . import model_registry


def _wrap(cfg, passes, joint=()):
    out = to_graph_trainer_config(cfg, model_registry)
    out.compile = GraphTrainerCompileConfig(enable=True, passes=list(passes), joint_passes=list(joint))
    return out


def graph_trainer_llama3_debugmodel():
    return _wrap(base.llama3_debugmodel(), ["transformer_block_bucketing"])


def graph_trainer_llama3_debugmodel_cudagraph():
    return _wrap(base.llama3_debugmodel(), ["transformer_block_bucketing", "cudagraph"], joint=["apply_sac"])


def graph_trainer_llama3_8b():
    return _wrap(base.llama3_8b(), ["auto_bucketing"], joint=["apply_sac", "fsdp_reshard_after_fwd"])
