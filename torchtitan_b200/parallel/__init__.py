"""Parallelism layer: rank-grid arithmetic, FSDP/HSDP/DDP runtime, TP/SP, CP, EP, PP and
activation checkpointing. The model code is single-device; these modules are applied to it
from the outside by each model's ``parallelize_fn``."""

from .parallel_dims import ParallelDims

__all__ = ["ParallelDims"]
