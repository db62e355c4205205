"""Hugging Face dataset glue. ``DatasetConfig`` = where the data lives, how to open it, and
how to turn a sample into text (torchtitan/hf_datasets/__init__.py:14-18)."""

from dataclasses import dataclass
from typing import Callable


@dataclass
class DatasetConfig:
    path: str
    loader: Callable
    sample_processor: Callable
