"""FLUX job configurations (torchtitan/models/flux/config_registry.py)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, TrainingConfig

from . import model_registry
from .flux_datasets import FluxDataLoader
from .trainer import Encoder, FluxTrainer
from .validate import FluxValidator


def flux_debugmodel() -> FluxTrainer.Config:
    return FluxTrainer.Config(
        metrics=MetricsProcessor.Config(log_freq=1), model_spec=model_registry("flux-debug"), tokenizer=None,
        dataloader=FluxDataLoader.Config(dataset="synthetic", img_size=64, t5_max_length=16, clip_max_length=16),
        optimizer=OptimizersContainer.Config(lr=8e-4), lr_scheduler=LRSchedulersContainer.Config(warmup_steps=1, decay_ratio=0.0),
        training=TrainingConfig(local_batch_size=4, seq_len=16, steps=10, max_norm=2.0),
        encoder=Encoder(random_init=True), checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
        validator=FluxValidator.Config(steps=2, timesteps=2, freq=5, dataloader=FluxDataLoader.Config(
            dataset="synthetic", img_size=64, t5_max_length=16, clip_max_length=16)),
    )


def _full(flavor: str) -> FluxTrainer.Config:
    return FluxTrainer.Config(
        metrics=MetricsProcessor.Config(log_freq=10), model_spec=model_registry(flavor), tokenizer=None,
        dataloader=FluxDataLoader.Config(dataset="cc12m-wds", img_size=256, t5_max_length=256),
        optimizer=OptimizersContainer.Config(lr=1e-4), lr_scheduler=LRSchedulersContainer.Config(warmup_steps=3000, decay_ratio=0.0),
        training=TrainingConfig(local_batch_size=32, seq_len=512, steps=30000, max_norm=2.0),
        encoder=Encoder(t5_encoder="google/t5-v1_1-xxl"), checkpoint=CheckpointManager.Config(interval=1000),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
    )


def flux_dev() -> FluxTrainer.Config:
    return _full("flux-dev")


def flux_schnell() -> FluxTrainer.Config:
    return _full("flux-schnell")
