"""DeepSeek-V3 job configurations (names as in torchtitan/models/deepseek_v3/config_registry.py:28-135)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.components.quantization.float8 import Float8GroupedMMConverter, Float8LinearConverter
from torchtitan_b200.config import ActivationCheckpointConfig, CompileConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.protocols.model_converter import ModelConvertersContainer
from torchtitan_b200.trainer import Trainer

from . import model_registry

_SAC_OP = dict(mode="selective", selective_ac_option="op")


def deepseek_v3_debugmodel() -> Trainer.Config:
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
        activation_checkpoint=ActivationCheckpointConfig(**_SAC_OP),
    )


def deepseek_v3_debugmodel_flex_attn() -> Trainer.Config:
    config = deepseek_v3_debugmodel()
    config.model_spec = model_registry("debugmodel_flex_attn")
    return config


def deepseek_v3_16b() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./assets/hf/deepseek-moe-16b-base",
        model_spec=model_registry("16B"),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=2.2e-4),
        lr_scheduler=LRSchedulersContainer.Config(decay_ratio=0.8, decay_type="cosine", min_lr_factor=0.1),
        training=TrainingConfig(local_batch_size=4, seq_len=4096, steps=1000),
        parallelism=ParallelismConfig(pipeline_parallel_schedule="Interleaved1F1B", expert_parallel_degree=8,
                                      expert_tensor_parallel_degree=1),
        checkpoint=CheckpointManager.Config(interval=10),
        activation_checkpoint=ActivationCheckpointConfig(**_SAC_OP),
        compile=CompileConfig(enable=True, components=["loss"]),
    )


def deepseek_v3_671b() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./assets/hf/DeepSeek-V3.1-Base",
        model_spec=model_registry("671B"),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=2.2e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2000, decay_ratio=0.8, decay_type="cosine", min_lr_factor=0.1),
        training=TrainingConfig(local_batch_size=4, seq_len=4096, steps=10000),
        parallelism=ParallelismConfig(pipeline_parallel_schedule="Interleaved1F1B", expert_parallel_degree=1,
                                      expert_tensor_parallel_degree=1),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(**_SAC_OP),
        compile=CompileConfig(enable=True, components=["loss"]),
        model_converters=ModelConvertersContainer.Config(converters=[
            Float8LinearConverter.Config(filter_fqns=["output", "router.gate"]),
            Float8GroupedMMConverter.Config(fqns=["experts"]),
        ]),
    )
