"""Configurations whose parallel layout is chosen by the planner for the visible world size
(names follow torchtitan/experiments/autoparallel/*/config_registry.py)."""

import os

from torchtitan_b200.models.deepseek_v3 import config_registry as dsv3
from torchtitan_b200.models.llama3 import config_registry as llama3

from .planner import auto_plan


def _apply(cfg):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    m = cfg.model_spec.model
    with __import__("torch").device("meta"):
        model = m.build()
    nparams, flops = m.get_nparams_and_flops(model, cfg.training.seq_len)
    plan = auto_plan(nparams, flops, m.n_layers, m.dim, cfg.training.seq_len, cfg.training.local_batch_size, world)
    cfg.parallelism.data_parallel_shard_degree = plan.dp_shard
    cfg.parallelism.tensor_parallel_degree = plan.tp
    cfg.parallelism.fsdp_reshard_after_forward = plan.reshard_after_forward
    cfg.activation_checkpoint.mode = plan.ac_mode
    return cfg


def autoparallel_llama3_debugmodel():
    return _apply(llama3.llama3_debugmodel())


def autoparallel_llama3_8b():
    return _apply(llama3.llama3_8b())


def autoparallel_deepseek_v3_debugmodel():
    return _apply(dsv3.deepseek_v3_debugmodel())
