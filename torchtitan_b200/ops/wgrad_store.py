"""Deferred weight gradients of linear layers, for pipeline schedules that split a backward step.

A zero-bubble schedule runs the backward of a (stage, micro-batch) in two actions: ``I`` forms the gradient of the
stage input (the next message of the pipeline) and ``W`` forms the weight gradients, at a later point where the rank
would otherwise wait. The reference gets the split from ``torch.distributed.pipelining`` (its ``stage_backward_input``
/ ``stage_backward_weight`` walk the autograd graph; torchtitan/distributed/pipeline_parallel.py:48-130 only picks the
schedule class). Here the split lives where the two halves separate naturally: a linear layer's backward is two
independent GEMMs, ``dx = dy @ W`` and ``dW = dy^T @ x``. While the runtime is inside an ``I`` action
(:meth:`WeightGradStore.collect`), :class:`_SplitLinearFn` computes ``dx`` only and parks a closure that holds ``dy``
and ``x``; the ``W`` action runs the parked closures, which accumulate into ``weight.grad``.

A weight is deferred when it is an autograd leaf (a plain ``nn.Parameter``, also a local tensor-parallel shard), or
when it is the gathered copy an FSDP / replicate unit handed out: the unit tags its copies with ``_wgrad_sink = (unit,
index)``, the parked closure puts its result into the unit's box for that backward pass, and the unit queues its
reduce-scatter behind the closures (``parallel/fsdp.py::_park_post_backward``), so ``W`` ends with one reduction of the
complete gradients. Any other non-leaf weight gets its gradient at once. Everything that is not a linear layer (norm
weights, embeddings, expert GEMMs, quantised linears) is also computed inside ``I``: those are a few percent of a dense
transformer's backward.
"""

from __future__ import annotations

import contextlib

import torch

__all__ = ["WeightGradStore", "split_linear"]


class WeightGradStore:
    #: set by the pipeline runtime when its schedule has separate ``I`` / ``W`` actions
    enabled: bool = False
    _open: list | None = None

    @classmethod
    def collecting(cls) -> bool:
        return cls._open is not None

    @classmethod
    def put(cls, fn) -> None:
        cls._open.append(fn)

    @classmethod
    @contextlib.contextmanager
    def collect(cls):
        """Everything deferred while this context is open lands in the yielded list (in backward order)."""
        assert cls._open is None, "input-gradient actions do not nest"
        cls._open = q = []
        try:
            yield q
        finally:
            cls._open = None

    @staticmethod
    def run(queue: list) -> None:
        with torch.no_grad():
            for fn in queue:
                fn()
        queue.clear()


def _native(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1
            and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0 and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0)


def _rows2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.stride(-1) == 1 else x2.contiguous()


def _mm(a, b, a_mn: bool, b_mn: bool, native: bool):
    """``op(a) @ op(b)^T`` in the convention of the framework's GEMM: ``a_mn`` means ``a`` is stored [K, M],
    ``b_mn`` means ``b`` is stored [K, N] (otherwise [N, K])."""
    if native:
        return torch.ops.tt_b200.gemm(a, b, a_mn, b_mn, False)
    return (a.t() if a_mn else a) @ (b if b_mn else b.t())


class _SplitLinearFn(torch.autograd.Function):
    """``y = x @ w^T (+ bias)`` whose weight gradient can be parked. ``leaf`` is the parameter that owns ``.grad``:
    ``w`` itself, or the fp32 parameter of which ``w`` is the autocast copy."""

    @staticmethod
    def forward(ctx, x, w, bias, leaf, sink=None):
        x2 = _rows2d(x)
        native = _native(x2, w)
        if native:
            from . import cuda_ops  # noqa: F401  (registers tt_b200::gemm)
        y = _mm(x2, w, False, False, native)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(x2, w)
        ctx.native, ctx.has_bias, ctx.xshape, ctx.leaf, ctx.sink = native, bias is not None, x.shape, leaf, sink
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = _rows2d(gy)
        native, leaf = ctx.native, ctx.leaf
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = _mm(g2, w, False, True, native).view(ctx.xshape)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = g2.float().sum(0).to(gy.dtype)
        if ctx.needs_input_grad[1]:
            if ctx.sink is not None and WeightGradStore.collecting():
                unit, index = ctx.sink
                box = unit.wgrad_box()

                def weight_grad_to_unit(g2=g2, x2=x2, box=box, index=index, native=native):
                    gw = _mm(g2, x2, True, True, native)
                    box[index] = gw if index not in box else box[index] + gw
                WeightGradStore.put(weight_grad_to_unit)
            elif leaf is not None and WeightGradStore.collecting():
                def weight_grad(g2=g2, x2=x2, leaf=leaf, native=native):
                    gw = _mm(g2, x2, True, True, native)
                    if leaf.grad is None:
                        leaf.grad = gw.to(leaf.dtype)
                    else:
                        leaf.grad.add_(gw)
                WeightGradStore.put(weight_grad)
            else:
                gw = _mm(g2, x2, True, True, native)
        return gx, gw, gb, None, None


def split_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Linear layer for runs with :attr:`WeightGradStore.enabled`; same values as the ordinary path."""
    leaf = weight if (weight.is_leaf and weight.requires_grad and type(weight) in (torch.Tensor, torch.nn.Parameter)) else None
    sink = getattr(weight, "_wgrad_sink", None) if leaf is None else None
    if x.is_cuda and torch.is_autocast_enabled() and weight.dtype == torch.float32:
        x, w = x.to(torch.bfloat16), weight.to(torch.bfloat16)
        bias = None if bias is None else bias.to(torch.bfloat16)
        return _SplitLinearFn.apply(x, w, bias, leaf, None)
    return _SplitLinearFn.apply(x, weight, bias, leaf, sink)
