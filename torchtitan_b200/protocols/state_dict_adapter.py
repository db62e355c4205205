"""State-dict adapters translate between this framework's parameter names/layouts and the
Hugging Face checkpoint of the same model.

Parity: torchtitan/protocols/state_dict_adapter.py:20-120. ``StateDictAdapter`` reads
``model.safetensors.index.json`` (when present under ``hf_assets_path``) into
``fqn_to_index_mapping`` so a multi-file HF export reproduces the original file split.
"""

from __future__ import annotations

import json
import os
import re
from abc import ABC, abstractmethod
from typing import Any

from torchtitan_b200.tools.logging import logger


class BaseStateDictAdapter(ABC):
    fqn_to_index_mapping: dict[Any, int] | None
    hf_assets_path: str | None

    @abstractmethod
    def __init__(self, model_config, hf_assets_path: str | None): ...

    @abstractmethod
    def to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]: ...

    @abstractmethod
    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]: ...

    @abstractmethod
    def get_hf_storage_reader(self, path: str, from_quantized: bool = False): ...


class StateDictAdapter(BaseStateDictAdapter):
    def __init__(self, model_config, hf_assets_path: str | None):
        self.model_config = model_config
        self.hf_assets_path = hf_assets_path
        self.fqn_to_index_mapping = None
        if hf_assets_path:
            index = os.path.join(hf_assets_path, "model.safetensors.index.json")
            try:
                with open(index) as f:
                    weight_map = json.load(f)["weight_map"]
            except FileNotFoundError:
                logger.warning(
                    f"model.safetensors.index.json not found at hf_assets_path: {index}. "
                    "Defaulting to saving a single safetensors file if checkpoint is saved in HF format"
                )
                weight_map = None
            if weight_map:
                self.fqn_to_index_mapping = {}
                for name, fname in weight_map.items():
                    m = re.search(r"\d+", fname)
                    if m:
                        self.fqn_to_index_mapping[name] = int(m.group(0))

    def get_hf_storage_reader(self, path: str, from_quantized: bool = False):
        if from_quantized:
            logger.warning("Loading from quantized checkpoint format is not supported for this model.")
        from torch.distributed.checkpoint import HuggingFaceStorageReader

        return HuggingFaceStorageReader(path)
