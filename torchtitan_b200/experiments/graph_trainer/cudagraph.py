"""CUDA-graph capture of a callable with static input buffers.

Parity: torchtitan/experiments/graph_trainer/cudagraph.py:23-170 (one shared graph memory pool and capture stream;
a wrapper that warms up, captures on the next call, copies non-static inputs into the captured buffers, checks that
static inputs keep their addresses, and replays). The callable here is an ordinary Python function launching this
framework's kernels -- e.g. the forward + backward of a training step -- not an FX graph module."""

from __future__ import annotations

from typing import Any, Callable, Sequence

import torch

_POOL = None
_STREAM = None


def init_global_graph_pool():
    """One memory pool and one capture stream shared by every wrapper of the process."""
    global _POOL, _STREAM
    if _POOL is None:
        _POOL = torch.cuda.graph_pool_handle()
        _STREAM = torch.cuda.Stream()
    return _POOL, _STREAM


class CUDAGraphWrapper:
    def __init__(self, runnable: Callable, example_inputs: Sequence[Any] | None = None, static_input_indices: Sequence[int] = (),
                 should_check_address: bool = False, warmup: int = 2, enabled: bool | None = None):
        self.runnable = runnable
        self.static = set(static_input_indices)
        self.check_address = should_check_address
        self.warmup_left = warmup
        self.enabled = torch.cuda.is_available() if enabled is None else enabled
        self.graph = None
        self.args: list[Any] | None = None
        self.output = None
        self.replays = 0

    def check_input_types(self, inputs) -> None:
        for x in inputs:
            if not isinstance(x, (torch.Tensor, int, float, bool, type(None), torch.Generator)):
                raise TypeError(f"args must be tensor, integer (for dynamic shapes), Generator (for random number generator), "
                                f"None, float or bool, but found {type(x)}")

    def copy_non_static_inputs(self, *args) -> None:
        for i, (dst, src) in enumerate(zip(self.args, args)):
            if i in self.static or not isinstance(src, torch.Tensor):
                continue
            if dst.shape != src.shape:
                raise RuntimeError(f"input {i} changed shape {tuple(dst.shape)} -> {tuple(src.shape)}: a captured graph is "
                                   "valid for one set of shapes")
            dst.copy_(src, non_blocking=True)

    def check_static_inputs_address(self, args) -> None:
        for i in self.static:
            if isinstance(args[i], torch.Tensor) and args[i].data_ptr() != self.args[i].data_ptr():
                raise RuntimeError(f"Static input {i} has a different address than at capture time")

    def __call__(self, *args):
        if not self.enabled:
            return self.runnable(*args)
        self.check_input_types(args)
        if self.warmup_left > 0:
            self.warmup_left -= 1
            return self.runnable(*args)
        if self.graph is None:
            pool, stream = init_global_graph_pool()
            self.args = [a if (i in self.static or not isinstance(a, torch.Tensor)) else a.clone() for i, a in enumerate(args)]
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, pool=pool, stream=stream):
                self.output = self.runnable(*self.args)
            torch.cuda.synchronize()
        if self.check_address:
            self.check_static_inputs_address(args)
        self.copy_non_static_inputs(*args)
        self.graph.replay()
        self.replays += 1
        return self.output
