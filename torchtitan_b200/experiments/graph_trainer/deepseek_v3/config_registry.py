"""Graph-trainer job configurations for DeepSeek-V3 (the names of
torchtitan/experiments/graph_trainer/deepseek_v3/config_registry.py:26-55). As for Llama 3, each job names its plan
passes; activation checkpointing stays as the base job sets it (the reference switches it off, because its tracer
cannot see through the checkpoint wrapper; the plan passes here work on the wrapped model)."""

from torchtitan_b200.experiments.graph_trainer.configs import GraphTrainerCompileConfig, to_graph_trainer_config
from torchtitan_b200.models.deepseek_v3 import config_registry as base

from . import model_registry


def _wrap(cfg, passes, joint=()):
    out = to_graph_trainer_config(cfg, model_registry)
    out.compile = GraphTrainerCompileConfig(enable=True, passes=list(passes), joint_passes=list(joint))
    return out


def graph_trainer_deepseek_v3_debugmodel():
    return _wrap(base.deepseek_v3_debugmodel(), ["transformer_block_bucketing"])


def graph_trainer_deepseek_v3_debugmodel_flex_attn():
    return _wrap(base.deepseek_v3_debugmodel_flex_attn(), ["transformer_block_bucketing"])


def graph_trainer_deepseek_v3_16b():
    return _wrap(base.deepseek_v3_16b(), ["auto_bucketing"], joint=["apply_sac"])


def graph_trainer_deepseek_v3_671b():
    return _wrap(base.deepseek_v3_671b(), ["auto_bucketing"], joint=["apply_sac"])
