"""Configurations whose parallel layout is chosen by the planner for the visible world size
(names follow torchtitan/experiments/autoparallel/*/config_registry.py)."""

import os

from torchtitan_b200.models.deepseek_v3 import config_registry as dsv3
from torchtitan_b200.models.llama3 import config_registry as llama3

from .planner import search, shape_of


def _apply(cfg):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    m = cfg.model_spec.model
    with __import__("torch").device("meta"):
        model = m.build()
    plans = search(shape_of(m, model, cfg.training.seq_len), cfg.training.seq_len, cfg.training.local_batch_size, world, keep=1)
    if not plans:
        raise RuntimeError(f"no parallel layout of {world} GPUs holds this model; add nodes")
    plan = plans[0]
    p = cfg.parallelism
    p.data_parallel_replicate_degree, p.data_parallel_shard_degree = plan.dp_replicate, plan.dp_shard
    p.tensor_parallel_degree, p.context_parallel_degree = plan.tp, plan.cp
    p.pipeline_parallel_degree, p.expert_parallel_degree = plan.pp, plan.ep
    if plan.pp > 1:
        p.pipeline_parallel_schedule = plan.pp_schedule
    p.fsdp_reshard_after_forward = plan.reshard_after_forward
    cfg.activation_checkpoint.mode = plan.ac_mode
    return cfg


def autoparallel_llama3_debugmodel():
    return _apply(llama3.llama3_debugmodel())


def autoparallel_llama3_8b():
    return _apply(llama3.llama3_8b())


def autoparallel_deepseek_v3_debugmodel():
    return _apply(dsv3.deepseek_v3_debugmodel())
