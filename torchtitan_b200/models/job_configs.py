"""One builder for the text pre-training job configurations of all model families.

A job configuration is mostly numbers (batch, sequence length, steps, learning rate, schedule, checkpoint interval,
parallel degrees). The registries of the families state those numbers as one call of :func:`text_job` per job; sections
that a job does not mention keep the defaults of ``Trainer.Config``. ``tests/test_reference_parity.py`` compares every
job, option by option, with the reference's configuration of the same name."""

from __future__ import annotations

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.components.validate import Validator
from torchtitan_b200.config import ActivationCheckpointConfig, CompileConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.protocols.model_converter import ModelConvertersContainer
from torchtitan_b200.tools.profiling import ProfilingConfig
from torchtitan_b200.trainer import Trainer

TEST_ASSETS = "./tests/assets/tokenizer"
DEBUG_SCHEDULE = dict(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0)


def text_job(spec, *, assets: str, dataset: str, lr: float, batch: int, seq: int, steps: int, schedule: dict | None = None,
             metrics: dict | None = None, profile_every: int | None = None, checkpoint: dict | None = None,
             ac: tuple[str, str] | str = ("selective", "op"), parallel: dict | None = None, compile: dict | None = None,
             converters: list | None = None, validate: tuple[int, int] | None = None, training: dict | None = None,
             optimizer: dict | None = None, config_cls=Trainer.Config, **extra_sections) -> Trainer.Config:
    """``spec``: the family's ``model_registry(flavor)``. ``assets``: tokenizer / checkpoint folder. ``schedule``,
    ``metrics``, ``checkpoint``, ``parallel``, ``compile``, ``training``: keyword arguments of the respective section.
    ``ac``: ``(mode, selective option)`` or a bare mode. ``validate``: ``(frequency, steps)``. ``profile_every``: profiler
    on, at this frequency. ``converters``: model converter configurations. ``optimizer``: further optimizer options.
    ``config_cls`` / ``extra_sections``: a trainer subclass' configuration and its own sections."""
    sections = dict(
        hf_assets_path=assets, model_spec=spec, dataloader=HuggingFaceTextDataLoader.Config(dataset=dataset),
        optimizer=OptimizersContainer.Config(lr=lr, **(optimizer or {})),
        training=TrainingConfig(local_batch_size=batch, seq_len=seq, steps=steps, **(training or {})),
        activation_checkpoint=(ActivationCheckpointConfig(mode=ac) if isinstance(ac, str)
                               else ActivationCheckpointConfig(mode=ac[0], selective_ac_option=ac[1])),
    )
    if schedule is not None:
        sections["lr_scheduler"] = LRSchedulersContainer.Config(**schedule)
    if metrics is not None:
        sections["metrics"] = MetricsProcessor.Config(**metrics)
    if profile_every is not None:
        sections["profiling"] = ProfilingConfig(enable_profiling=True, profile_freq=profile_every)
    if checkpoint is not None:
        sections["checkpoint"] = CheckpointManager.Config(**checkpoint)
    if parallel is not None:
        sections["parallelism"] = ParallelismConfig(**parallel)
    if compile is not None:
        sections["compile"] = CompileConfig(**compile)
    if converters is not None:
        sections["model_converters"] = ModelConvertersContainer.Config(converters=list(converters))
    if validate is not None:
        sections["validator"] = Validator.Config(freq=validate[0], steps=validate[1])
    return config_cls(**sections, **extra_sections)


def debug_job(spec, **changes) -> Trainer.Config:
    """The ten-step debug job on the offline test data: batch 8 x 2048 tokens, lr 8e-4, warm-up 2 then linear decay to
    zero, logging every step, a checkpoint at the end, selective checkpointing of every second layer."""
    settings = dict(assets=TEST_ASSETS, dataset="c4_test", lr=8e-4, batch=8, seq=2048, steps=10, schedule=DEBUG_SCHEDULE,
                    metrics=dict(log_freq=1), checkpoint=dict(interval=10, last_save_model_only=False), ac=("selective", "2"))
    settings.update(changes)
    return text_job(spec, **settings)
