"""Data loader base classes.

Parity: torchtitan/components/dataloader.py:32-167. ``ParallelAwareDataloader`` wraps
torchdata's ``StatefulDataLoader``; its checkpoint state is ``{"dp_rank_<r>": pickle(state),
"world_size": dp_world_size}`` and loading with a different data-parallel degree is refused.
``SyntheticDataLoader`` (an addition) produces seeded uniform random token batches in pinned
host memory, for benchmarks and for runs without a dataset.
"""

from __future__ import annotations

import inspect
import pickle
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Iterator

import torch
from torch.distributed.checkpoint.stateful import Stateful
from torch.utils.data import IterableDataset
from torchdata.stateful_dataloader import StatefulDataLoader

from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.tools.logging import logger


class DataloaderExhaustedError(Exception):
    """The iterator ran out of data; the Trainer ends the run cleanly when it sees this."""


class BaseDataLoader(Stateful, ABC, Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        dataset: str = ""
        dataset_path: str | None = None

    @abstractmethod
    def __iter__(self) -> Iterator[tuple[dict[str, torch.Tensor], torch.Tensor]]: ...


class ParallelAwareDataloader(StatefulDataLoader, BaseDataLoader):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseDataLoader.Config):
        num_workers: int = 0
        persistent_workers: bool = False
        pin_memory: bool = False
        prefetch_factor: int | None = None

    dp_rank: int
    dp_world_size: int

    def __init__(self, dataset: IterableDataset, dp_rank: int, dp_world_size: int, **kwargs):
        self._validate_kwargs(kwargs)
        self.dp_world_size = dp_world_size
        self.dp_rank = dp_rank
        self._rank_id = f"dp_rank_{dp_rank}"
        super().__init__(dataset, **kwargs)

    @staticmethod
    def _validate_kwargs(kwargs: dict[str, Any]) -> None:
        if "dataset" in kwargs:
            raise ValueError("'dataset' should not be passed in kwargs; it must be provided as the first positional argument.")
        valid = frozenset(n for n in inspect.signature(StatefulDataLoader.__init__).parameters if n not in ("self", "dataset"))
        bad = set(kwargs) - valid
        if bad:
            raise ValueError(f"Invalid dataloader kwargs: {bad}. Valid kwargs are: {sorted(valid)}")
        if kwargs.get("num_workers", 0) == 0:
            kwargs.pop("persistent_workers", None)
            kwargs.pop("prefetch_factor", None)

    def state_dict(self) -> dict[str, Any]:
        return {self._rank_id: pickle.dumps(super().state_dict()), "world_size": self.dp_world_size}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        if not state_dict:
            return
        if self._rank_id not in state_dict:
            logger.warning(f"DataLoader state is empty for dp rank {self.dp_rank}, expected key {self._rank_id}")
            return
        assert self.dp_world_size == state_dict["world_size"], (
            "dp_degree is inconsistent before and after checkpoint, dataloader resharding is not supported yet."
        )
        super().load_state_dict(pickle.loads(state_dict[self._rank_id]))


class SyntheticDataLoader(BaseDataLoader):
    """Uniform random tokens: ``input`` int64 [local_batch, seq_len] over ``[0, vocab)``, labels =
    inputs shifted left by one (the last label is drawn too). Rank ``r`` uses seed
    ``seed + r`` so data differs across data-parallel ranks; the state is the batch counter."""

    @dataclass(kw_only=True, slots=True)
    class Config(BaseDataLoader.Config):
        dataset: str = "synthetic"
        seed: int = 0
        vocab_size: int | None = None
        """Defaults to the model's vocabulary."""
        pin_memory: bool = True
        num_batches: int | None = None

    def __init__(self, config: Config, *, dp_world_size: int, dp_rank: int, tokenizer=None, seq_len: int,
                 local_batch_size: int, model_vocab_size: int | None = None, **kwargs):
        self.config = config
        self.dp_rank, self.dp_world_size = dp_rank, dp_world_size
        self.seq_len, self.batch = seq_len, local_batch_size
        self.vocab = config.vocab_size or model_vocab_size or (tokenizer.get_vocab_size() if tokenizer is not None else None)
        assert self.vocab, "SyntheticDataLoader needs a vocab size"
        self._n = 0
        self._pin = config.pin_memory and torch.cuda.is_available()

    def _make(self, idx: int):
        g = torch.Generator().manual_seed((self.config.seed + self.dp_rank) * 1_000_003 + idx)
        x = torch.randint(0, self.vocab, (self.batch, self.seq_len + 1), generator=g, dtype=torch.int64)
        inp, lab = x[:, :-1].contiguous(), x[:, 1:].contiguous()
        if self._pin:
            inp, lab = inp.pin_memory(), lab.pin_memory()
        return {"input": inp}, lab

    def __iter__(self):
        while self.config.num_batches is None or self._n < self.config.num_batches:
            out = self._make(self._n)
            self._n += 1
            yield out

    def state_dict(self):
        return {f"dp_rank_{self.dp_rank}": pickle.dumps({"n": self._n}), "world_size": self.dp_world_size}

    def load_state_dict(self, state_dict):
        key = f"dp_rank_{self.dp_rank}"
        if not state_dict or key not in state_dict:
            return
        assert self.dp_world_size == state_dict["world_size"]
        self._n = pickle.loads(state_dict[key])["n"]
