"""Device dispatch for the hot ops: CUDA tensors go to the native kernels (autograd wrappers
in ``ops/cuda_ops.py``), everything else to the PyTorch definitions."""

from __future__ import annotations

import torch

from . import reference as ref
from .wgrad_store import WeightGradStore, split_linear


def native_available() -> bool:
    from . import native

    return native.available()


def _cuda(x) -> bool:
    return x.is_cuda


def linear(x, weight, bias=None):
    if WeightGradStore.enabled and weight.requires_grad and torch.is_grad_enabled():
        return split_linear(x, weight, bias)   # a pipeline schedule with separate weight-gradient actions is running
    if _cuda(x):
        from . import cuda_ops

        return cuda_ops.linear(x, weight, bias)
    return ref.linear(x, weight, bias)


def rms_norm(x, weight, eps: float):
    if _cuda(x):
        from . import cuda_ops

        return cuda_ops.rms_norm(x, weight, eps)
    return ref.rms_norm(x, weight, eps)


def rope(x, table, positions=None, layout: str = "interleaved"):
    if _cuda(x):
        from . import cuda_ops

        return cuda_ops.rope(x, table, positions, layout)
    return ref.rope(x, table, positions, layout)


def swiglu(gate, up):
    if _cuda(gate):
        from . import cuda_ops

        return cuda_ops.swiglu(gate, up)
    return ref.swiglu(gate, up)


def attention(q, k, v, *, causal=True, scale=None, window=None, doc_ids=None, sinks=None, return_lse=False):
    if _cuda(q):
        from . import cuda_ops

        return cuda_ops.attention(
            q, k, v, causal=causal, scale=scale, window=window, doc_ids=doc_ids, sinks=sinks, return_lse=return_lse
        )
    return ref.attention(
        q, k, v, causal=causal, scale=scale, window=window, doc_ids=doc_ids, sinks=sinks, return_lse=return_lse
    )


def cross_entropy_sum(logits, labels, ignore_index: int = -100):
    if _cuda(logits):
        from . import cuda_ops

        return cuda_ops.cross_entropy_sum(logits, labels, ignore_index)
    return ref.cross_entropy_sum(logits, labels, ignore_index)


def token_logprobs(logits, labels):
    if _cuda(logits):
        from . import cuda_ops

        return cuda_ops.token_logprobs(logits, labels)
    return ref.token_logprobs(logits, labels)
