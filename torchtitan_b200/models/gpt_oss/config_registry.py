"""gpt-oss job configurations (names as in torchtitan/models/gpt_oss/config_registry.py:23-140)."""

from torchtitan_b200.models import job_configs as _jobs
from torchtitan_b200.trainer import Trainer

from . import model_registry

_NO_EXPERT_PARALLEL = dict(expert_parallel_degree=1, expert_tensor_parallel_degree=1)


def gpt_oss_debugmodel() -> Trainer.Config:
    return _jobs.debug_job(model_registry("debugmodel"), ac=("none", "2"), parallel=_NO_EXPERT_PARALLEL, validate=(5, 10))


def _sized(flavor: str, folder: str) -> Trainer.Config:
    return _jobs.text_job(model_registry(flavor), assets=f"./assets/hf/{folder}", dataset="c4", lr=8e-4, batch=1, seq=8192, steps=10000,
                    schedule=dict(warmup_steps=2000, decay_ratio=0.8, decay_type="cosine", min_lr_factor=0.1),
                    checkpoint=dict(interval=500), ac="full", parallel=_NO_EXPERT_PARALLEL)


def gpt_oss_20b() -> Trainer.Config:
    return _sized("20b", "gpt-oss-20b")


def gpt_oss_120b() -> Trainer.Config:
    return _sized("120b", "gpt-oss-120b")
