"""Data parallel modes of the graph trainer on top of the framework's FSDP runtime.

The reference implements ``replicate`` / ``fully_shard`` / ``hybrid_shard`` as DTensor parametrisations that a
compiler later buckets and reorders (torchtitan/experiments/graph_trainer/simple_fsdp.py:28-317). Here the three modes
select meshes for the same flat-buffer runtime, and the plan decides how parameters are bucketed into units."""

from __future__ import annotations

import torch
import torch.nn as nn

from torchtitan_b200.parallel import fsdp
from torchtitan_b200.parallel.fsdp import MixedPrecisionPolicy

from .passes import StepPlan


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


def data_parallel(model: nn.Module, mesh, mode: str = "fully_shard", mp_policy: MixedPrecisionPolicy | None = None,
                  plan: StepPlan | None = None) -> nn.Module:
    assert mode in ("replicate", "fully_shard", "hybrid_shard"), f"Unsupported mode {mode}"
    plan = plan or StepPlan()
    mp = mp_policy or MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    if mode == "replicate":
        fsdp.replicate(model, mesh=mesh, mp_policy=mp)
        return model
    if mode == "hybrid_shard":
        assert mesh.ndim == 2, "hybrid_shard needs a (replicate, shard) mesh"
    raf = {"default": None, "always": True, "never": False}[plan.reshard_after_forward]
    buckets = auto_buckets(model, plan.bucket_bytes) if plan.bucketing == "auto" else get_transformer_block_buckets(model)
    for b in buckets:
        mods = [model.get_submodule(n) for n in ([b] if isinstance(b, str) else b)]
        fsdp.fully_shard(mods if len(mods) > 1 else mods[0], mesh=mesh, mp_policy=mp,
                         reshard_after_forward=True if raf is None else raf)
    fsdp.fully_shard(model, mesh=mesh, mp_policy=mp, reshard_after_forward=True if raf is None else raf)
    return model
