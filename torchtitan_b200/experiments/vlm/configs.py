"""Trainer configuration of the vision-language experiment: the common one with the multimodal loader as the
``--dataloader.*`` section, so that its options (``max_images_per_batch``, ``max_patches_per_image``,
``packing_buffer_size`` ...) are addressable from the command line (torchtitan/experiments/vlm/configs.py:15-19)."""

from __future__ import annotations

from dataclasses import dataclass, field

from torchtitan_b200.trainer import Trainer

from .datasets import MMDataLoader


@dataclass(kw_only=True, slots=True)
class MultiModalTrainerConfig(Trainer.Config):
    dataloader: MMDataLoader.Config = field(default_factory=MMDataLoader.Config)
