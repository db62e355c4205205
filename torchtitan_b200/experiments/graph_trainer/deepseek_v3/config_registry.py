"""Graph-trainer job configurations for DeepSeek-V3."""

from torchtitan_b200.experiments.graph_trainer.configs import GraphTrainerCompileConfig, to_graph_trainer_config
from torchtitan_b200.models.deepseek_v3 import config_registry as base

from . import model_registry


def graph_trainer_deepseek_v3_debugmodel():
    out = to_graph_trainer_config(base.deepseek_v3_debugmodel(), model_registry)
    out.compile = GraphTrainerCompileConfig(enable=True, passes=["transformer_block_bucketing"])
    return out


def graph_trainer_deepseek_v3_16b():
    out = to_graph_trainer_config(base.deepseek_v3_16b(), model_registry)
    out.compile = GraphTrainerCompileConfig(enable=True, passes=["auto_bucketing"], joint_passes=["apply_sac"])
    return out
