"""``llama3_ft_debugmodel``: the Llama-3 debug job with the fault-tolerant trainer, as a DiLoCo run of 100 steps that
synchronises two model fragments every 10 steps (the settings of torchtitan/experiments/ft/llama3/config_registry.py:21-66).
``--fault_tolerance.process_group gloo`` runs the replica groups' traffic on CPU ranks."""

from torchtitan_b200.config import CommConfig
from torchtitan_b200.experiments.ft.config import FaultTolerance
from torchtitan_b200.experiments.ft.optimizer import FTOptimizersContainer
from torchtitan_b200.experiments.ft.trainer import FaultTolerantTrainer
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.models import job_configs as _jobs
from torchtitan_b200.models.llama3 import model_registry
from torchtitan_b200.tools.profiling import ProfilingConfig


def llama3_ft_debugmodel() -> FaultTolerantTrainer.Config:
    cfg = _jobs.debug_job(
        model_registry("debugmodel"), steps=100, validate=(5, 10), config_cls=FaultTolerantTrainer.Config,
        profiling=ProfilingConfig(enable_profiling=True, profile_freq=10, profiler_active=10, profiler_warmup=0),
        comm=CommConfig(train_timeout_seconds=15),
        fault_tolerance=FaultTolerance(enable=True, semi_sync_method="diloco", process_group="nccl", process_group_timeout_ms=10000,
                                       sync_steps=10, num_fragments=2))
    cfg.optimizer = FTOptimizersContainer.Config(lr=8e-4)
    cfg.dataloader = HuggingFaceTextDataLoader.Config()
    return cfg
