"""Qwen3 job configurations. Names follow torchtitan/models/qwen3/config_registry.py:22-225;
``qwen3_30b_a3b`` (EP=8 with expert-bias balancing and per-step router histograms) and the
``*_synthetic`` variants are additions."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.dataloader import SyntheticDataLoader
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.trainer import Trainer

from . import model_registry


def _debug(flavor: str) -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./tests/assets/tokenizer",
        metrics=MetricsProcessor.Config(log_freq=1),
        model_spec=model_registry(flavor),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4_test"),
        optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(local_batch_size=8, seq_len=2048, steps=10),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="2"),
    )


def qwen3_debugmodel() -> Trainer.Config:
    return _debug("debugmodel")


def qwen3_debugmodel_flex() -> Trainer.Config:
    return _debug("debugmodel_flex")


def _sized(flavor: str, hf: str, lr: float, bs: int, seq: int, steps: int, *, warmup: int = 600, interval: int = 500,
           ac: str = "selective", log_freq: int = 10, **par) -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path=f"./assets/hf/{hf}",
        metrics=MetricsProcessor.Config(log_freq=log_freq),
        model_spec=model_registry(flavor),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=lr),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=warmup),
        training=TrainingConfig(local_batch_size=bs, seq_len=seq, steps=steps),
        parallelism=ParallelismConfig(**par),
        checkpoint=CheckpointManager.Config(interval=interval, last_save_model_only=False, export_dtype="float16"),
        activation_checkpoint=ActivationCheckpointConfig(mode=ac, selective_ac_option="op"),
    )


def qwen3_0_6b() -> Trainer.Config:
    return _sized("0.6B", "Qwen3-0.6B", 3e-4, 4, 4096, 10, warmup=2, log_freq=1)


def qwen3_1_7b() -> Trainer.Config:
    return _sized("1.7B", "Qwen3-1.7B", 8e-4, 4, 4096, 100, warmup=20, interval=50)


def qwen3_14b() -> Trainer.Config:
    return _sized("14B", "Qwen3-14B", 8e-4, 4, 4096, 3000, ac="full", tensor_parallel_degree=1)


def qwen3_32b() -> Trainer.Config:
    return _sized("32B", "Qwen3-32B", 8e-4, 2, 4096, 3000, ac="full", tensor_parallel_degree=1)


def qwen3_moe_debug() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./tests/assets/tokenizer",
        metrics=MetricsProcessor.Config(log_freq=1),
        model_spec=model_registry("debugmodel_moe"),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4_test"),
        optimizer=OptimizersContainer.Config(lr=3e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2),
        training=TrainingConfig(local_batch_size=4, seq_len=4096, steps=10),
        parallelism=ParallelismConfig(expert_parallel_degree=1, expert_tensor_parallel_degree=1),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False, export_dtype="float16"),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="op"),
    )


def _synthetic(cfg: Trainer.Config) -> Trainer.Config:
    cfg.tokenizer = None
    cfg.dataloader = SyntheticDataLoader.Config(seed=0)
    return cfg


def qwen3_debugmodel_synthetic() -> Trainer.Config:
    return _synthetic(qwen3_debugmodel())


def qwen3_moe_debug_synthetic() -> Trainer.Config:
    cfg = _synthetic(qwen3_moe_debug())
    cfg.model_spec = model_registry("debugmodel_moe", balance_experts=True)
    return cfg


def qwen3_30b_a3b() -> Trainer.Config:
    """Qwen3-30B-A3B, EP=8 on one 8-GPU node: local batch 1 x 4096, synthetic tokens, expert-bias
    balancing (step 1e-3) and a per-step token-per-expert histogram in the metrics."""
    cfg = Trainer.Config(
        hf_assets_path="./assets/hf/Qwen3-30B-A3B",
        metrics=MetricsProcessor.Config(log_freq=1, log_moe_histogram=True),
        model_spec=model_registry("30B-A3B", balance_experts=True),
        optimizer=OptimizersContainer.Config(lr=3e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=200, decay_ratio=0.1),
        training=TrainingConfig(local_batch_size=1, seq_len=4096, steps=1000),
        parallelism=ParallelismConfig(expert_parallel_degree=8),
        checkpoint=CheckpointManager.Config(interval=500),
        # no activation checkpointing: 114 GB of 180 at this batch, and about twice the throughput of per-op selective
        # checkpointing, which replays every token exchange (and its buffer-size read on the host) in the backward pass
        activation_checkpoint=ActivationCheckpointConfig(mode="none"),
    )
    return _synthetic(cfg)


def qwen3_30b_a3b_mxfp8() -> Trainer.Config:
    """The same job with the routed experts' three grouped GEMMs in MXFP8 (forward, input gradient and weight gradient,
    each one grouped launch with the group boundaries on the device); attention, router and output stay bf16.
    Parity: torchtitan/components/quantization/mx.py:91-134 (``MXFP8Converter`` on ``fqns = ["experts"]``)."""
    from torchtitan_b200.components.quantization.mx import MXFP8Converter
    from torchtitan_b200.protocols.model_converter import ModelConvertersContainer

    cfg = qwen3_30b_a3b()
    cfg.model_converters = ModelConvertersContainer.Config(converters=[MXFP8Converter.Config(fqns=["experts"])])
    return cfg

