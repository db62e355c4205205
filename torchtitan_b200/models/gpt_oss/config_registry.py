"""gpt-oss job configurations (names as in torchtitan/models/gpt_oss/config_registry.py:23-140)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.components.validate import Validator
from torchtitan_b200.config import ActivationCheckpointConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.trainer import Trainer

from . import model_registry


def gpt_oss_debugmodel() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./tests/assets/tokenizer",
        metrics=MetricsProcessor.Config(log_freq=1),
        model_spec=model_registry("debugmodel"),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4_test"),
        optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(local_batch_size=8, seq_len=2048, steps=10),
        parallelism=ParallelismConfig(expert_parallel_degree=1, expert_tensor_parallel_degree=1),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="none", selective_ac_option="2"),
        validator=Validator.Config(freq=5, steps=10),
    )


def _sized(flavor: str, assets: str) -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path=f"./assets/hf/{assets}",
        model_spec=model_registry(flavor),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2000, decay_ratio=0.8, decay_type="cosine", min_lr_factor=0.1),
        training=TrainingConfig(local_batch_size=1, seq_len=8192, steps=10000),
        parallelism=ParallelismConfig(expert_parallel_degree=1, expert_tensor_parallel_degree=1),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
    )


def gpt_oss_20b() -> Trainer.Config:
    return _sized("20b", "gpt-oss-20b")


def gpt_oss_120b() -> Trainer.Config:
    return _sized("120b", "gpt-oss-120b")
