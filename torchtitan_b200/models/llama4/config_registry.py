"""Llama 4 job configurations (names as in torchtitan/models/llama4/config_registry.py:21-109)."""

from torchtitan_b200.models import job_configs as _jobs
from torchtitan_b200.trainer import Trainer

from . import model_registry

_ADAM = dict(eps=1e-15)


def llama4_debugmodel() -> Trainer.Config:
    return _jobs.debug_job(model_registry("debugmodel"), lr=4e-3, optimizer=_ADAM, schedule={**_jobs.DEBUG_SCHEDULE, "min_lr_factor": 0.1},
                     ac=("selective", "op"), parallel=dict(expert_parallel_degree=1, expert_tensor_parallel_degree=1))


def _large(flavor: str, folder: str, batch: int, **degrees) -> Trainer.Config:
    return _jobs.text_job(model_registry(flavor), assets=f"./assets/hf/{folder}", dataset="c4", lr=4e-3, optimizer=_ADAM, batch=batch,
                    seq=8192, steps=3000, schedule=dict(warmup_steps=600, min_lr_factor=0.1), checkpoint=dict(interval=500),
                    ac="full", parallel=dict(tensor_parallel_degree=8, expert_parallel_degree=1, expert_tensor_parallel_degree=8,
                                             **degrees))


def llama4_17bx128e() -> Trainer.Config:
    return _large("17bx128e", "Llama-4-Maverick-17B-128E", 1, pipeline_parallel_degree=4)


def llama4_17bx16e() -> Trainer.Config:
    return _large("17bx16e", "Llama-4-Scout-17B-16E", 8)
