"""``llama3_ft_debugmodel``: the Llama-3 debug job with the fault-tolerant trainer
(torchtitan/experiments/ft/llama3/config_registry.py:21-66)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, TrainingConfig
from torchtitan_b200.experiments.ft.config import FaultTolerance
from torchtitan_b200.experiments.ft.trainer import FaultTolerantTrainer
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.models.llama3 import model_registry


def llama3_ft_debugmodel() -> FaultTolerantTrainer.Config:
    return FaultTolerantTrainer.Config(
        hf_assets_path="./tests/assets/tokenizer",
        metrics=MetricsProcessor.Config(log_freq=1),
        model_spec=model_registry("debugmodel"),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4_test"),
        optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(local_batch_size=8, seq_len=2048, steps=10),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="2"),
        fault_tolerance=FaultTolerance(enable=True, process_group="gloo", group_size=2, min_replica_size=1),
    )
