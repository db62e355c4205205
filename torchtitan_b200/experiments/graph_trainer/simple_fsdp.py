"""Bucket layouts of the graph trainer's data parallelism.

The reference implements ``replicate`` / ``fully_shard`` / ``hybrid_shard`` as DTensor parametrisations that a
compiler later buckets and reorders (torchtitan/experiments/graph_trainer/simple_fsdp.py:28-317). Here the three modes
are the meshes of the framework's flat-buffer FSDP runtime (chosen by the parallelism degrees, as for every trainer),
and what the compiler passes decide is how blocks are grouped into units: ``GraphTrainer`` hands the plan's bucket size
to ``parallel/data_parallel.py::apply_fsdp``, which groups consecutive blocks the way :func:`auto_buckets` lists them."""

from __future__ import annotations

import torch.nn as nn


def get_transformer_block_buckets(model: nn.Module) -> list[list[str] | str]:
    """Bucket names: [embedding], one per block, [final norm, output] (graph_trainer/common_utils.py:100-128)."""
    buckets: list[list[str] | str] = []
    if getattr(model, "tok_embeddings", None) is not None:
        buckets.append("tok_embeddings")
    buckets += [f"layers.{k}" for k in model.layers.keys()]
    tail = [n for n in ("norm", "output") if getattr(model, n, None) is not None]
    if tail:
        buckets.append(tail)
    return buckets


def auto_buckets(model: nn.Module, bucket_bytes: int, elem_size: int = 2) -> list[list[str] | str]:
    """Greedy grouping of consecutive blocks until a bucket's gathered size reaches ``bucket_bytes``."""
    out: list[list[str] | str] = []
    if getattr(model, "tok_embeddings", None) is not None:
        out.append("tok_embeddings")
    cur, size = [], 0
    for k, blk in model.layers.items():
        n = sum(p.numel() for p in blk.parameters()) * elem_size
        if cur and size + n > bucket_bytes:
            out.append(cur)
            cur, size = [], 0
        cur.append(f"layers.{k}")
        size += n
    if cur:
        out.append(cur)
    tail = [n for n in ("norm", "output") if getattr(model, n, None) is not None]
    if tail:
        out.append(tail)
    return out
