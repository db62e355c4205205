"""Integration tests: lists of command-line override sets, each run as real training jobs through ``run_train.sh``.

Reference: tests/integration_tests/__init__.py:16-31 (the ``OverrideDefinitions`` record users extend for their own
suites). One definition may hold several override sets; they run one after another in the same dump folder, which is
how save-then-resume cases are written."""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

__all__ = ["OverrideDefinitions"]


@dataclass
class OverrideDefinitions:
    override_args: Sequence[Sequence[str]] = ((),)
    test_descr: str = "default"
    test_name: str = "default"
    ngpu: int = 4
    disabled: bool = False
    needs_gpu: bool = False
    """The case exercises a CUDA-only path (float8 / MXFP8 kernels, peer-memory collectives): skipped on CPU runs."""
    module: str = "llama3"
    config: str = "llama3_debugmodel"
    env: Sequence[dict] = ()
    """Extra environment of override set ``i`` (``env[i]``), e.g. ``{"TRAIN_FILE": ...}`` to launch another entry point
    such as the FLUX inference script on the checkpoint the first set saved."""

    def __repr__(self) -> str:
        return self.test_descr

    def flags(self, i: int) -> list[str]:
        """Override set ``i`` as an argv list (each entry may hold a flag and its value separated by a space)."""
        out: list[str] = []
        for entry in self.override_args[i]:
            out.extend(entry.split())
        return out
