"""Configuration layer: ``Configurable`` base, shared dataclasses and the CLI manager.

Parity: torchtitan/config/__init__.py:9-13 (dtype map), configurable.py, configs.py, manager.py.
"""

import torch

from .configurable import Configurable
from .configs import (
    ActivationCheckpointConfig,
    CommConfig,
    CompileConfig,
    DebugConfig,
    ParallelismConfig,
    TrainingConfig,
)

TORCH_DTYPE_MAP = {
    "float16": torch.float16,
    "float32": torch.float32,
    "bfloat16": torch.bfloat16,
}

__all__ = [
    "Configurable",
    "TORCH_DTYPE_MAP",
    "TrainingConfig",
    "ParallelismConfig",
    "ActivationCheckpointConfig",
    "CompileConfig",
    "CommConfig",
    "DebugConfig",
    "ConfigManager",
]


def __getattr__(name):
    # ConfigManager imports tyro, keep that import lazy.
    if name == "ConfigManager":
        from .manager import ConfigManager

        return ConfigManager
    raise AttributeError(name)
