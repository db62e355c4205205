"""Text datasets packed into fixed-length training windows.

Parity: torchtitan/hf_datasets/text_datasets.py:35-217 -- datasets ``c4`` (streamed),
``c4_test`` (local ``tests/assets/c4_test``) and ``c4_validation``; each sample is encoded with
BOS and EOS, appended to a rolling token buffer, and windows of ``seq_len + 1`` tokens are cut
off as ``({"input": x[:-1]}, x[1:])``; samples are split over data-parallel ranks with
``split_dataset_by_node``; the checkpoint state is the token buffer plus either the sample index
(map-style) or the streaming dataset's own state; ``infinite`` re-loops.
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import partial
from typing import Any

import torch
from torch.distributed.checkpoint.stateful import Stateful
from torch.utils.data import IterableDataset

from torchtitan_b200.components.dataloader import ParallelAwareDataloader
from torchtitan_b200.tools.logging import logger

from . import DatasetConfig


def _open_c4(path: str, split: str):
    from datasets import load_dataset

    return load_dataset(path, name="en", split=split, streaming=True)


def _open_local(path: str):
    from datasets import load_dataset

    return load_dataset(path, split="train")


def _c4_text(sample: dict[str, Any]) -> str:
    return sample["text"]


DATASETS = {
    "c4": DatasetConfig(path="allenai/c4", loader=partial(_open_c4, split="train"), sample_processor=_c4_text),
    "c4_test": DatasetConfig(path="tests/assets/c4_test", loader=_open_local, sample_processor=_c4_text),
    "c4_validation": DatasetConfig(path="allenai/c4", loader=partial(_open_c4, split="validation"), sample_processor=_c4_text),
}


def _validate_dataset(name: str, path: str | None = None):
    if name not in DATASETS:
        raise ValueError(f"Dataset {name} is not supported. Supported datasets are: {list(DATASETS.keys())}")
    cfg = DATASETS[name]
    path = path or cfg.path
    logger.info(f"Preparing {name} dataset from {path}")
    return path, cfg.loader, cfg.sample_processor


class HuggingFaceTextDataset(IterableDataset, Stateful):
    def __init__(self, dataset_name: str, dataset_path: str | None, tokenizer, seq_len: int = 2048,
                 dp_rank: int = 0, dp_world_size: int = 1, infinite: bool = False) -> None:
        from datasets.distributed import split_dataset_by_node

        dataset_name = dataset_name.lower()
        path, loader, to_text = _validate_dataset(dataset_name, dataset_path)
        self.dataset_name = dataset_name
        self._data = split_dataset_by_node(loader(path), dp_rank, dp_world_size)
        self._tokenizer = tokenizer
        self.seq_len = seq_len
        self.infinite = infinite
        self._to_text = to_text
        self._sample_idx = 0
        self._token_buffer: list[int] = []

    def _is_map_style(self) -> bool:
        from datasets import Dataset

        return isinstance(self._data, Dataset)

    def _samples(self):
        if self._is_map_style():
            if self._sample_idx == len(self._data):
                return iter(())
            return iter(self._data.skip(self._sample_idx))
        return iter(self._data)

    def __iter__(self):
        window = self.seq_len + 1
        while True:
            for sample in self._samples():
                self._token_buffer.extend(self._tokenizer.encode(self._to_text(sample), add_bos=True, add_eos=True))
                self._sample_idx += 1
                while len(self._token_buffer) >= window:
                    x = torch.LongTensor(self._token_buffer[:window])
                    self._token_buffer = self._token_buffer[window:]
                    yield {"input": x[:-1]}, x[1:]
            if not self.infinite:
                logger.warning(f"Dataset {self.dataset_name} has run out of data")
                return
            self._sample_idx = 0
            logger.warning(f"Dataset {self.dataset_name} is being re-looped")
            if not self._is_map_style() and hasattr(self._data, "set_epoch") and hasattr(self._data, "epoch"):
                self._data.set_epoch(self._data.epoch + 1)

    def state_dict(self):
        sd: dict[str, Any] = {"token_buffer": self._token_buffer}
        if self._is_map_style():
            sd["sample_idx"] = self._sample_idx
        else:
            sd["data"] = self._data.state_dict()
        return sd

    def load_state_dict(self, state_dict):
        self._token_buffer = state_dict["token_buffer"]
        if self._is_map_style():
            self._sample_idx = state_dict["sample_idx"]
        else:
            assert "data" in state_dict
            self._data.load_state_dict(state_dict["data"])


class HuggingFaceTextDataLoader(ParallelAwareDataloader):
    @dataclass(kw_only=True, slots=True)
    class Config(ParallelAwareDataloader.Config):
        dataset: str = "c4_test"
        infinite: bool = True

    def __init__(self, config: Config, *, dp_world_size: int, dp_rank: int, tokenizer, seq_len: int,
                 local_batch_size: int, **kwargs):
        ds = HuggingFaceTextDataset(
            dataset_name=config.dataset, dataset_path=config.dataset_path, tokenizer=tokenizer, seq_len=seq_len,
            dp_rank=dp_rank, dp_world_size=dp_world_size, infinite=config.infinite,
        )
        super().__init__(
            ds, dp_rank=dp_rank, dp_world_size=dp_world_size, num_workers=config.num_workers,
            persistent_workers=config.persistent_workers, pin_memory=config.pin_memory,
            prefetch_factor=config.prefetch_factor, batch_size=local_batch_size,
        )
