"""Job configurations for Llama-3 (``--module llama3 --config <function name>``).

Function names and settings follow torchtitan/models/llama3/config_registry.py:30-216.
``llama3_8b_synthetic`` and ``llama3_debugmodel_synthetic`` are additions that need no dataset
or tokenizer (seeded random tokens)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.dataloader import SyntheticDataLoader
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer, OptimizersInBackwardContainer
from torchtitan_b200.components.quantization.float8 import Float8LinearConverter
from torchtitan_b200.components.validate import Validator
from torchtitan_b200.config import ActivationCheckpointConfig, CompileConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.protocols.model_converter import ModelConvertersContainer
from torchtitan_b200.tools.profiling import ProfilingConfig
from torchtitan_b200.trainer import Trainer

from . import model_registry


def llama3_debugmodel() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./tests/assets/tokenizer",
        model_spec=model_registry("debugmodel"),
        optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(local_batch_size=8, seq_len=2048, steps=10),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4_test"),
        metrics=MetricsProcessor.Config(log_freq=1),
        parallelism=ParallelismConfig(pipeline_parallel_schedule="Interleaved1F1B"),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="2"),
        validator=Validator.Config(freq=5, steps=10),
    )


def llama3_debugmodel_synthetic() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.tokenizer = None
    cfg.dataloader = SyntheticDataLoader.Config(seed=0)
    cfg.validator = Validator.Config(freq=5, steps=10, dataloader=SyntheticDataLoader.Config(seed=1))
    return cfg


def llama3_debugmodel_flex_attn() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.model_spec = model_registry("debugmodel_flex_attn")
    return cfg


def llama3_debugmodel_varlen_attn() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.model_spec = model_registry("debugmodel_varlen_attn")
    return cfg


def llama3_debugmodel_opt_in_bwd() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.optimizer = OptimizersInBackwardContainer.Config(lr=8e-4)
    return cfg


def llama3_debugmodel_float8() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.model_converters = ModelConvertersContainer.Config(converters=[
        Float8LinearConverter.Config(enable_fsdp_float8_all_gather=True, precompute_float8_dynamic_scale_for_fsdp=True),
    ])
    return cfg


def llama3_debugmodel_float8_emulate() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.model_converters = ModelConvertersContainer.Config(converters=[
        Float8LinearConverter.Config(enable_fsdp_float8_all_gather=True, precompute_float8_dynamic_scale_for_fsdp=True, emulate=True),
    ])
    return cfg


def llama3_8b() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./assets/hf/Llama-3.1-8B",
        profiling=ProfilingConfig(enable_profiling=True, profile_freq=100),
        metrics=MetricsProcessor.Config(enable_tensorboard=True),
        model_spec=model_registry("8B"),
        optimizer=OptimizersContainer.Config(lr=3e-4),
        training=TrainingConfig(local_batch_size=1, seq_len=8192, steps=1000),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4"),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="op"),
        validator=Validator.Config(freq=500, steps=1200),
    )


def llama3_8b_synthetic() -> Trainer.Config:
    """Llama-3.1-8B throughput job: synthetic tokens, warmup-stable-decay schedule, no profiler."""
    cfg = llama3_8b()
    cfg.tokenizer = None
    cfg.dataloader = SyntheticDataLoader.Config(seed=0)
    cfg.profiling = ProfilingConfig()
    cfg.metrics = MetricsProcessor.Config(log_freq=10)
    cfg.lr_scheduler = LRSchedulersContainer.Config(warmup_steps=200, decay_ratio=0.1, decay_type="linear")
    # per-op SAC keeps every matmul output when the device has the room (sharded runs on 180 GB parts do)
    cfg.activation_checkpoint.per_op_sac_mm_policy = "auto"
    return cfg


def llama3_8b_synthetic_mxfp8() -> Trainer.Config:
    """The throughput job with every transformer Linear in MXFP8 (e4m3 data, one E8M0 scale per 32 elements along the
    contraction, bf16 master copies, fp32 accumulation); the output projection stays bf16, as in
    torchtitan docs/mxfp8.md. Add ``--parallelism.tensor_parallel_degree 2 --parallelism.enable_async_tensor_parallel``
    for the FSDP x TP layout."""
    from torchtitan_b200.components.quantization.mx import MXFP8Converter

    cfg = llama3_8b_synthetic()
    cfg.model_converters = ModelConvertersContainer.Config(converters=[
        MXFP8Converter.Config(fqns=["attention", "feed_forward"]),
    ])
    return cfg


def llama3_70b() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./assets/hf/Llama-3.1-70B",
        profiling=ProfilingConfig(enable_profiling=True, profile_freq=100),
        metrics=MetricsProcessor.Config(enable_tensorboard=True),
        model_spec=model_registry("70B"),
        optimizer=OptimizersContainer.Config(lr=1.5e-4),
        training=TrainingConfig(local_batch_size=8, seq_len=8192, steps=1000),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4"),
        parallelism=ParallelismConfig(tensor_parallel_degree=8),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
        validator=Validator.Config(freq=500, steps=1200),
    )


def llama3_405b() -> Trainer.Config:
    return Trainer.Config(
        hf_assets_path="./assets/hf/Llama-3.1-405B",
        profiling=ProfilingConfig(enable_profiling=True, profile_freq=100),
        metrics=MetricsProcessor.Config(enable_tensorboard=True),
        model_spec=model_registry("405B"),
        model_converters=ModelConvertersContainer.Config(converters=[
            Float8LinearConverter.Config(
                enable_fsdp_float8_all_gather=True, precompute_float8_dynamic_scale_for_fsdp=True, filter_fqns=["output"],
            ),
        ]),
        optimizer=OptimizersContainer.Config(lr=8e-5),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=600),
        training=TrainingConfig(local_batch_size=2, seq_len=8192, steps=3000),
        dataloader=HuggingFaceTextDataLoader.Config(dataset="c4"),
        parallelism=ParallelismConfig(tensor_parallel_degree=8, enable_async_tensor_parallel=True),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
        compile=CompileConfig(enable=True),
        validator=Validator.Config(freq=500, steps=1200),
    )
