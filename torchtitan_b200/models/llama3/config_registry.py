"""Job configurations for Llama-3 (``--module llama3 --config <function name>``).

Function names and settings follow torchtitan/models/llama3/config_registry.py:30-216.
``llama3_8b_synthetic`` and ``llama3_debugmodel_synthetic`` are additions that need no dataset
or tokenizer (seeded random tokens)."""

from torchtitan_b200.components.dataloader import SyntheticDataLoader
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersInBackwardContainer
from torchtitan_b200.components.quantization.float8 import Float8LinearConverter
from torchtitan_b200.components.validate import Validator
from torchtitan_b200.models import job_configs as _jobs
from torchtitan_b200.protocols.model_converter import ModelConvertersContainer
from torchtitan_b200.tools.profiling import ProfilingConfig
from torchtitan_b200.trainer import Trainer

from . import model_registry

_FP8_ALL_GATHER = dict(enable_fsdp_float8_all_gather=True, precompute_float8_dynamic_scale_for_fsdp=True)


def _pretrain(flavor: str, folder: str, **job) -> Trainer.Config:
    """The C4 pre-training jobs: profiler every 100 steps, TensorBoard, checkpoints every 500 steps, validation every 500
    steps over 1200 batches."""
    job.setdefault("steps", 1000)
    return _jobs.text_job(model_registry(flavor), assets=f"./assets/hf/{folder}", dataset="c4", seq=8192, profile_every=100,
                    metrics=dict(enable_tensorboard=True), checkpoint=dict(interval=500), validate=(500, 1200), **job)


def llama3_debugmodel() -> Trainer.Config:
    return _jobs.debug_job(model_registry("debugmodel"), parallel=dict(pipeline_parallel_schedule="Interleaved1F1B"), validate=(5, 10))


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
        Float8LinearConverter.Config(**_FP8_ALL_GATHER),
    ])
    return cfg


def llama3_debugmodel_float8_emulate() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.model_converters = ModelConvertersContainer.Config(converters=[
        Float8LinearConverter.Config(emulate=True, **_FP8_ALL_GATHER),
    ])
    return cfg


def llama3_8b() -> Trainer.Config:
    return _pretrain("8B", "Llama-3.1-8B", lr=3e-4, batch=1)


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
    return _pretrain("70B", "Llama-3.1-70B", lr=1.5e-4, batch=8, ac="full", parallel=dict(tensor_parallel_degree=8))


def llama3_405b() -> Trainer.Config:
    return _pretrain("405B", "Llama-3.1-405B", lr=8e-5, batch=2, steps=3000, ac="full", schedule=dict(warmup_steps=600),
                     parallel=dict(tensor_parallel_degree=8, enable_async_tensor_parallel=True), compile=dict(enable=True),
                     converters=[Float8LinearConverter.Config(filter_fqns=["output"], **_FP8_ALL_GATHER)])
