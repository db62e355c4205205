"""Job configurations (names as in torchtitan/experiments/transformers_modeling_backend/config_registry.py:26-90)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, DebugConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.tools.profiling import ProfilingConfig

from . import model_registry
from .configs import TransformersBackendConfig


def _cfg(flavor: str, dataset: str, **kw) -> TransformersBackendConfig:
    return TransformersBackendConfig(
        hf_model="Qwen/Qwen3-4B-Instruct-2507", debug=DebugConfig(print_config=True), model_spec=model_registry(flavor),
        profiling=ProfilingConfig(profile_freq=5), optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(local_batch_size=2, seq_len=2048, steps=10),
        dataloader=HuggingFaceTextDataLoader.Config(dataset=dataset), metrics=MetricsProcessor.Config(log_freq=1),
        parallelism=ParallelismConfig(pipeline_parallel_schedule="1F1B"),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="2"), **kw,
    )


def transformers_modeling_backend_debugmodel() -> TransformersBackendConfig:
    return _cfg("debugmodel", "c4_test", hf_assets_path="./tests/assets/tokenizer")


def transformers_modeling_backend_full() -> TransformersBackendConfig:
    return _cfg("full", "c4")
