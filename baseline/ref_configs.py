"""Side module for running the *reference* on the benchmark config without datasets or a
tokenizer: ``--module baseline.ref_configs --config llama3_8b_synthetic`` (the reference's config
manager accepts fully-qualified module paths). Only a data loader is added; model, trainer,
parallelisation, optimizer and loss are the reference's own stock code."""

from __future__ import annotations

import pickle
from dataclasses import dataclass

import torch

from torchtitan.components.dataloader import BaseDataLoader
from torchtitan.models.llama3.config_registry import llama3_8b
from torchtitan.components.metrics import MetricsProcessor
from torchtitan.tools.profiling import ProfilingConfig


class SyntheticLoader(BaseDataLoader):
    """Uniform random tokens from seed 0 (+ data-parallel rank), pinned host batches."""

    @dataclass(kw_only=True, slots=True)
    class Config(BaseDataLoader.Config):
        dataset: str = "synthetic"
        seed: int = 0
        vocab_size: int = 128256

    def __init__(self, config: Config, *, dp_world_size: int, dp_rank: int, tokenizer=None, seq_len: int,
                 local_batch_size: int, **kwargs):
        self.c, self.rank, self.world, self.seq, self.bs, self.n = config, dp_rank, dp_world_size, seq_len, local_batch_size, 0

    def __iter__(self):
        while True:
            g = torch.Generator().manual_seed((self.c.seed + self.rank) * 1_000_003 + self.n)
            x = torch.randint(0, self.c.vocab_size, (self.bs, self.seq + 1), generator=g, dtype=torch.int64)
            self.n += 1
            inp, lab = x[:, :-1].contiguous(), x[:, 1:].contiguous()
            if torch.cuda.is_available():
                inp, lab = inp.pin_memory(), lab.pin_memory()
            yield {"input": inp}, lab

    def state_dict(self):
        return {f"dp_rank_{self.rank}": pickle.dumps({"n": self.n}), "world_size": self.world}

    def load_state_dict(self, sd):
        if sd and f"dp_rank_{self.rank}" in sd:
            self.n = pickle.loads(sd[f"dp_rank_{self.rank}"])["n"]


def llama3_8b_synthetic():
    cfg = llama3_8b()
    cfg.tokenizer = None
    cfg.dataloader = SyntheticLoader.Config()
    cfg.profiling = ProfilingConfig()
    cfg.metrics = MetricsProcessor.Config(log_freq=1000000)
    return cfg
