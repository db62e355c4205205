"""torch.profiler schedule and CUDA memory snapshots driven by ``ProfilingConfig``.

Parity: torchtitan/tools/profiling.py:22-213. Traces go to
``<dump>/<save_traces_folder>/iteration_<N>/rank<r>_trace.json``; memory snapshots to
``<dump>/<save_memory_snapshot_folder>/iteration_<N>/rank<r>_memory_snapshot.pickle`` and are
also written when a step dies with an out-of-memory error.
"""

from __future__ import annotations

import contextlib
import os
import pickle
import time
from dataclasses import dataclass

import torch

from .logging import logger

MEMORY_SNAPSHOT_MAX_ENTRIES = 100000


@dataclass(kw_only=True, slots=True)
class ProfilingConfig:
    enable_profiling: bool = False
    save_traces_folder: str = "profile_traces"
    profile_freq: int = 10
    profiler_active: int = 1
    profiler_warmup: int = 3
    profiler_repeat: int | None = None
    """How many wait/warm-up/active cycles to record (unset: every cycle until the run ends)."""
    profiler_skip_first: int | None = None
    """Steps to ignore before the first cycle starts."""
    profiler_skip_first_wait: int | None = None
    """Non-zero: the first cycle starts with its warm-up instead of its wait."""
    enable_memory_snapshot: bool = False
    save_memory_snapshot_folder: str = "memory_snapshot"
    experimental_cuda_device_timestamps: bool = False
    """*B200* also read the per-kernel device timestamps the fused kernels record."""


def _rank() -> int:
    return torch.distributed.get_rank() if torch.distributed.is_initialized() else 0


@contextlib.contextmanager
def maybe_enable_profiling(config: ProfilingConfig, *, global_step: int = 0, base_folder: str = "", leaf_folder: str = ""):
    if not config.enable_profiling:
        yield None
        return
    trace_dir = os.path.join(base_folder, config.save_traces_folder)
    freq, warmup, active = config.profile_freq, config.profiler_warmup, config.profiler_active
    rank = _rank()

    def on_ready(prof):
        out = os.path.join(trace_dir, f"iteration_{prof.step_num}", leaf_folder)
        os.makedirs(out, exist_ok=True)
        t0 = time.monotonic()
        prof.export_chrome_trace(os.path.join(out, f"rank{rank}_trace.json"))
        logger.info("Finished dumping profiler traces in %.2f seconds", time.monotonic() - t0)

    wait = freq - (active + warmup)
    assert wait >= 0, "profile_freq must be >= profiler_active + profiler_warmup"
    cycle = {k: v for k, v in (("repeat", config.profiler_repeat), ("skip_first", config.profiler_skip_first),
                                ("skip_first_wait", config.profiler_skip_first_wait)) if v is not None}
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    logger.info(f"Profiling active. Traces will be saved at {trace_dir}")
    os.makedirs(trace_dir, exist_ok=True)
    with torch.profiler.profile(
        activities=acts,
        schedule=torch.profiler.schedule(wait=wait, warmup=warmup, active=active, **cycle),
        on_trace_ready=on_ready,
        record_shapes=True,
    ) as prof:
        prof.step_num = global_step
        yield prof


class _MemorySnapshots:
    def __init__(self, folder: str, freq: int, global_step: int):
        self.folder, self.freq, self.step_num = folder, freq, global_step
        torch.cuda.memory._record_memory_history(max_entries=MEMORY_SNAPSHOT_MAX_ENTRIES)

    def step(self, exit_ctx: bool = False) -> None:
        self.step_num += 1
        if not exit_ctx and self.step_num % self.freq != 0:
            return
        name = f"iteration_{self.step_num - 1}_exit" if exit_ctx else f"iteration_{self.step_num}"
        out = os.path.join(self.folder, name)
        os.makedirs(out, exist_ok=True)
        t0 = time.monotonic()
        with open(os.path.join(out, f"rank{_rank()}_memory_snapshot.pickle"), "wb") as f:
            pickle.dump(torch.cuda.memory._snapshot(), f)
        logger.info("Finished dumping memory snapshot in %.2f seconds", time.monotonic() - t0)


@contextlib.contextmanager
def maybe_enable_memory_snapshot(config: ProfilingConfig, *, global_step: int = 0, base_folder: str = ""):
    if not (config.enable_memory_snapshot and torch.cuda.is_available()):
        yield None
        return
    folder = os.path.join(base_folder, config.save_memory_snapshot_folder)
    os.makedirs(folder, exist_ok=True)
    snap = _MemorySnapshots(folder, config.profile_freq, global_step)
    logger.info(f"Memory profiler active. Snapshot will be saved at {folder}")
    try:
        yield snap
    except torch.OutOfMemoryError:
        snap.step(exit_ctx=True)
        raise
