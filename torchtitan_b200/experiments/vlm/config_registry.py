"""Job configurations for the vision-language experiment (torchtitan/experiments/vlm/config_registry.py)."""

import dataclasses

from torchtitan_b200.components.validate import Validator
from torchtitan_b200.config import ParallelismConfig
from torchtitan_b200.models.llama3 import config_registry as _llama3

from . import model_registry
from .configs import MultiModalTrainerConfig
from .datasets import MMDataLoader


def vlm_debugmodel() -> MultiModalTrainerConfig:
    """The text debug job (optimizer, schedule, batch, checkpoint and checkpointing settings) with the vision-language
    model, the multimodal loader on the image-caption pairs of the ``cc12m-test`` shard under ``tests/assets``
    (``--dataloader.dataset synthetic`` needs no files at all), no validation and the default pipeline schedule."""
    text = _llama3.llama3_debugmodel()
    settings = {f.name: getattr(text, f.name) for f in dataclasses.fields(text)}
    settings.update(model_spec=model_registry("debugmodel"), dataloader=MMDataLoader.Config(dataset="cc12m-test"),
                    validator=Validator.Config(), parallelism=ParallelismConfig())
    return MultiModalTrainerConfig(**settings)
