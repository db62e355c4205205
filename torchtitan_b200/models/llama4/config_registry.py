"""Llama 4 job configurations (names as in torchtitan/models/llama4/config_registry.py:21-109)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.trainer import Trainer

from . import model_registry


def llama4_debugmodel() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./tests/assets/tokenizer",
        metrics=MetricsProcessor.Config(log_freq=1),
        model_spec=model_registry("debugmodel"),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4_test"),
        optimizer=OptimizersContainer.Config(lr=4e-3, eps=1e-15),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.1),
        training=TrainingConfig(local_batch_size=8, seq_len=2048, steps=10),
        parallelism=ParallelismConfig(expert_parallel_degree=1, expert_tensor_parallel_degree=1),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="op"),
    )


def _large(flavor: str, assets: str, batch: int, **par) -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path=f"./assets/hf/{assets}",
        model_spec=model_registry(flavor),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=4e-3, eps=1e-15),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=600, min_lr_factor=0.1),
        training=TrainingConfig(local_batch_size=batch, seq_len=8192, steps=3000),
        parallelism=ParallelismConfig(**par),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
    )


def llama4_17bx128e() -> Trainer.Config:
    return _large("17bx128e", "Llama-4-Maverick-17B-128E", 1, tensor_parallel_degree=8, pipeline_parallel_degree=4,
                  expert_parallel_degree=1, expert_tensor_parallel_degree=8)


def llama4_17bx16e() -> Trainer.Config:
    return _large("17bx16e", "Llama-4-Scout-17B-16E", 8, tensor_parallel_degree=8, expert_parallel_degree=1,
                  expert_tensor_parallel_degree=8)
