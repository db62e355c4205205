"""Graph-trainer job configurations for Llama 3 (the names of
torchtitan/experiments/graph_trainer/llama3/config_registry.py:25-52, plus a CUDA-graph variant of the debug job).

The reference leaves ``compile.passes`` empty and expects them on the command line; here each job names the plan passes
that suit its size (block-wise buckets for small models, automatic buckets with the selective-checkpoint and
reshard-after-forward joint passes from 8B up). ``--compile.passes`` / ``--compile.joint_passes`` replace them."""

from torchtitan_b200.experiments.graph_trainer.configs import GraphTrainerCompileConfig, to_graph_trainer_config
from torchtitan_b200.models.llama3 import config_registry as base

from . import model_registry

_SMALL = (["transformer_block_bucketing"], [])
_LARGE = (["auto_bucketing"], ["apply_sac", "fsdp_reshard_after_fwd"])


def _wrap(cfg, passes, joint=()):
    out = to_graph_trainer_config(cfg, model_registry)
    out.compile = GraphTrainerCompileConfig(enable=True, passes=list(passes), joint_passes=list(joint))
    return out


def graph_trainer_llama3_debugmodel():
    return _wrap(base.llama3_debugmodel(), *_SMALL)


def graph_trainer_llama3_debugmodel_flex_attn():
    return _wrap(base.llama3_debugmodel_flex_attn(), *_SMALL)


def graph_trainer_llama3_debugmodel_cudagraph():
    return _wrap(base.llama3_debugmodel(), ["transformer_block_bucketing", "cudagraph"], joint=["apply_sac"])


def graph_trainer_llama3_8b():
    return _wrap(base.llama3_8b(), *_LARGE)


def graph_trainer_llama3_70b():
    return _wrap(base.llama3_70b(), *_LARGE)


def graph_trainer_llama3_405b():
    return _wrap(base.llama3_405b(), *_LARGE)
