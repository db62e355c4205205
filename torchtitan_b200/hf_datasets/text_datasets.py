"""Text datasets packed into fixed-length training windows.

Behaviour of torchtitan/hf_datasets/text_datasets.py:35-217 -- datasets ``c4`` (streamed), ``c4_test`` (local
``tests/assets/c4_test``) and ``c4_validation``; samples are split over data-parallel ranks with
``split_dataset_by_node``, encoded with BOS and EOS and packed into windows of ``seq_len + 1`` tokens yielded as
``({"input": x[:-1]}, x[1:])``; the checkpoint state (keys ``token_buffer`` and ``sample_idx`` or ``data``) resumes the
stream exactly; ``infinite`` re-loops. Built here from three parts: a sample source per dataset kind (indexed /
streaming) that knows its own position, a packer that owns the rolling buffer and cuts all complete windows of a sample
at once, and the dataset that strings them together.
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


def register_dataset(name: str, config: DatasetConfig) -> None:
    """Make another text dataset available to ``--dataloader.dataset``."""
    DATASETS[name.lower()] = config


def _lookup(name: str, path: str | None):
    try:
        cfg = DATASETS[name]
    except KeyError:
        raise ValueError(f"Dataset {name} is not supported. Supported datasets are: {list(DATASETS.keys())}") from None
    logger.info(f"Preparing {name} dataset from {path or cfg.path}")
    return cfg, path or cfg.path


class _IndexedSource:
    """A map-style dataset shard: position = number of samples consumed (checkpoint key ``sample_idx``)."""

    def __init__(self, data):
        self.data, self.pos = data, 0

    def __iter__(self):
        remaining = self.data.skip(self.pos) if self.pos < len(self.data) else ()
        for sample in remaining:
            self.pos += 1
            yield sample

    def rewind(self) -> None:
        self.pos = 0

    def state(self) -> dict[str, Any]:
        return {"sample_idx": self.pos}

    def restore(self, state: dict[str, Any]) -> None:
        self.pos = state["sample_idx"]


class _StreamSource:
    """A streaming dataset shard: the position is whatever the stream reports about itself (checkpoint key ``data``)."""

    def __init__(self, data):
        self.data = data

    def __iter__(self):
        return iter(self.data)

    def rewind(self) -> None:
        if hasattr(self.data, "set_epoch") and hasattr(self.data, "epoch"):
            self.data.set_epoch(self.data.epoch + 1)     # a new epoch reshuffles the shards

    def state(self) -> dict[str, Any]:
        return {"data": self.data.state_dict()}

    def restore(self, state: dict[str, Any]) -> None:
        assert "data" in state, "checkpoint of a streaming dataset lacks the stream position"
        self.data.load_state_dict(state["data"])


class _Packer:
    """Rolling token buffer cut into windows of ``seq_len + 1`` tokens; a window gives inputs ``[:-1]`` and labels ``[1:]``."""

    def __init__(self, seq_len: int):
        self.window = seq_len + 1
        self.tokens: list[int] = []

    def feed(self, ids):
        self.tokens.extend(ids)
        cut = len(self.tokens) - len(self.tokens) % self.window
        if not cut:
            return
        full, self.tokens = torch.tensor(self.tokens[:cut], dtype=torch.long).view(-1, self.window), self.tokens[cut:]
        pending = full.unbind(0)
        for k, row in enumerate(pending):
            # a consumer that checkpoints between two windows of one sample must find the later windows in the buffer
            rest = [t for r in pending[k + 1:] for t in r.tolist()]
            saved, self.tokens = self.tokens, rest + self.tokens
            yield {"input": row[:-1]}, row[1:]
            self.tokens = saved


class HuggingFaceTextDataset(IterableDataset, Stateful):
    """Samples of this data-parallel rank -> text -> tokens (BOS ... EOS) -> packed windows. Checkpoint state: the
    packer's left-over tokens plus the source position."""

    def __init__(self, dataset_name: str, dataset_path: str | None, tokenizer, seq_len: int = 2048,
                 dp_rank: int = 0, dp_world_size: int = 1, infinite: bool = False) -> None:
        from datasets import Dataset
        from datasets.distributed import split_dataset_by_node

        self.dataset_name = dataset_name.lower()
        cfg, path = _lookup(self.dataset_name, dataset_path)
        shard = split_dataset_by_node(cfg.loader(path), dp_rank, dp_world_size)
        self._source = _IndexedSource(shard) if isinstance(shard, Dataset) else _StreamSource(shard)
        self._to_text, self._tokenizer = cfg.sample_processor, tokenizer
        self._packer = _Packer(seq_len)
        self.seq_len, self.infinite = seq_len, infinite

    def __iter__(self):
        while True:
            for sample in self._source:
                yield from self._packer.feed(self._tokenizer.encode(self._to_text(sample), add_bos=True, add_eos=True))
            if not self.infinite:
                logger.warning(f"Dataset {self.dataset_name} has run out of data")
                return
            logger.warning(f"Dataset {self.dataset_name} is being re-looped")
            self._source.rewind()

    def state_dict(self):
        return {"token_buffer": list(self._packer.tokens), **self._source.state()}

    def load_state_dict(self, state_dict):
        self._packer.tokens = list(state_dict["token_buffer"])
        self._source.restore(state_dict)


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
