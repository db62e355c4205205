"""Job configurations for the vision-language experiment (torchtitan/experiments/vlm/config_registry.py)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, TrainingConfig
from . import model_registry
from .configs import MultiModalTrainerConfig
from .datasets import MMDataLoader


def vlm_debugmodel() -> MultiModalTrainerConfig:
    """Image-caption pairs of the ``cc12m-test`` shard under ``tests/assets`` (``--dataloader.dataset synthetic`` needs no
    files at all)."""
    return MultiModalTrainerConfig(
        hf_assets_path="./tests/assets/tokenizer", metrics=MetricsProcessor.Config(log_freq=1),
        model_spec=model_registry("debugmodel"),
        dataloader=MMDataLoader.Config(dataset="cc12m-test"), optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(local_batch_size=8, seq_len=2048, steps=10),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="2"),
    )
