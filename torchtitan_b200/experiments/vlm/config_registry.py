"""Job configurations for the vision-language experiment (torchtitan/experiments/vlm/config_registry.py)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, TrainingConfig
from torchtitan_b200.trainer import Trainer

from . import model_registry
from .datasets import MMDataLoader


def vlm_debugmodel() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./tests/assets/tokenizer", metrics=MetricsProcessor.Config(log_freq=1),
        model_spec=model_registry("debugmodel"),
        dataloader=MMDataLoader.Config(dataset="synthetic", max_patches_per_image=16, max_images_per_batch=128), optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(local_batch_size=4, seq_len=512, steps=10),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="2"),
    )
