"""Apply FSDP / HSDP / DDP to a decoder the way the reference groups parameters
(torchtitan/models/llama3/parallelize.py:340-405): one unit for ``tok_embeddings``, one per
transformer block, one for ``[norm, output]`` (kept gathered after forward because backward
starts there), and a root unit for anything left."""

from __future__ import annotations

import torch
import torch.nn as nn

from torchtitan_b200.tools.logging import logger

from .fsdp import MixedPrecisionPolicy, fully_shard, replicate
from .fsdp_policy import get_fsdp_reshard_after_forward_policy


def make_comm(dp_mesh, parallelism, model=None, param_dtype=torch.bfloat16):
    """Pick the transport for FSDP collectives: NVLink peer-memory kernels when every rank of the
    shard mesh is a CUDA device of this host and the option is on, else c10d."""
    if parallelism is not None and not getattr(parallelism, "fused_fsdp_collectives", True):
        return None
    if not torch.cuda.is_available() or dp_mesh is None:
        return None
    try:
        from .nvlink_comm import NvlinkComm

        return NvlinkComm.maybe_create(dp_mesh, model=model, param_dtype=param_dtype)
    except ImportError:
        return None


def _compute_copy_bytes(model: nn.Module, dtype: torch.dtype) -> int:
    return sum(p.numel() for p in model.parameters()) * torch.empty((), dtype=dtype).element_size()


def apply_fsdp(model: nn.Module, dp_mesh, param_dtype: torch.dtype, reduce_dtype: torch.dtype, pp_enabled: bool,
               cpu_offload: bool = False, reshard_after_forward_policy: str = "default", parallelism=None,
               extra_groups: dict | None = None, efsdp_mesh=None):
    mp = MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype)
    reshard = get_fsdp_reshard_after_forward_policy(
        reshard_after_forward_policy, pp_enabled, param_bytes=_compute_copy_bytes(model, param_dtype)
    )
    compute_device = None
    if cpu_offload:
        # sharded parameters, gradients and optimizer state stay in (pinned) host memory; every gather starts with a
        # host-to-device copy of the shard, every reduce-scatter ends with a device-to-host copy, the optimizer runs on
        # the CPU (torchtitan/models/llama3/parallelize.py:334, ``CPUOffloadPolicy``). Collectives go through c10d.
        compute_device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        logger.info(f"FSDP CPU offload: shards in host memory, compute on {compute_device}")
    comm = None if cpu_offload else make_comm(dp_mesh, parallelism, model=model, param_dtype=param_dtype)
    if comm is None and getattr(parallelism, "fsdp_extra_process_group", False) and dp_mesh is not None:
        import torch.distributed as dist

        from .fsdp import C10dComm

        shard_mesh = dp_mesh[dp_mesh.mesh_dim_names[-1]] if dp_mesh.ndim == 2 else dp_mesh
        # new_group is collective over the whole job: every rank creates every shard group and keeps its own
        ranks_mine = dist.get_process_group_ranks(shard_mesh.get_group())
        all_sets = [None] * dist.get_world_size()
        dist.all_gather_object(all_sets, tuple(ranks_mine))
        own = None
        for ranks in sorted(set(all_sets)):
            g = dist.new_group(list(ranks))
            if tuple(ranks_mine) == ranks:
                own = g
        comm = C10dComm(gather_group=own)
        logger.info("FSDP all-gathers use a process group of their own")
    kw = dict(mesh=dp_mesh, mp_policy=mp, comm=comm, compute_device=compute_device)
    if getattr(model, "tok_embeddings", None) is not None:
        fully_shard(model.tok_embeddings, **kw, reshard_after_forward=reshard)
    bucket_bytes = int(getattr(parallelism, "fsdp_bucket_bytes", 0) or 0)
    elem = torch.empty((), dtype=param_dtype).element_size()
    group, group_bytes = [], 0

    def flush():
        nonlocal group, group_bytes
        if group:
            fully_shard(group if len(group) > 1 else group[0], **kw, reshard_after_forward=reshard)
        group, group_bytes = [], 0

    for block in model.layers.values():
        if efsdp_mesh is not None and getattr(block, "moe_enabled", False):
            # MoE-aware FSDP: expert-parallel weights are only replicated over the efsdp ranks
            fully_shard(block.moe.experts, mesh=efsdp_mesh, mp_policy=mp, reshard_after_forward=reshard,
                        compute_device=compute_device)
        if bucket_bytes <= 0:
            fully_shard(block, **kw, reshard_after_forward=reshard)
            continue
        # bucketed units: consecutive blocks share one unit (one gather / one reduce for the whole group)
        n = sum(p.numel() for p in block.parameters()) * elem
        if group and group_bytes + n > bucket_bytes:
            flush()
        group.append(block)
        group_bytes += n
    flush()
    if getattr(model, "norm", None) is not None and getattr(model, "output", None) is not None:
        fully_shard([model.norm, model.output], **kw, reshard_after_forward=reshard_after_forward_policy == "always")
    fully_shard(model, **kw, reshard_after_forward=reshard)
    from .fsdp import fsdp_units

    depth = max(int(getattr(parallelism, "fsdp_prefetch_depth", 1) or 1), 1)
    units = fsdp_units(model)
    for u in units:
        u.prefetch_depth = depth
    logger.info(f"FSDP: {len(units)} units, reshard_after_forward={reshard}, prefetch depth {depth}, "
                f"transport={'nvlink' if comm is not None and type(comm).__name__ == 'NvlinkComm' else 'c10d'}")
    return model


def apply_replicate(model: nn.Module, dp_mesh, param_dtype: torch.dtype, reduce_dtype: torch.dtype):
    mp = MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype)
    kw = dict(mesh=dp_mesh, mp_policy=mp)
    if getattr(model, "tok_embeddings", None) is not None:
        replicate(model.tok_embeddings, **kw)
    for block in model.layers.values():
        replicate(block, **kw)
    if getattr(model, "norm", None) is not None and getattr(model, "output", None) is not None:
        replicate([model.norm, model.output], **kw)
    replicate(model, **kw)
    logger.info("Applied replicate to the model")
    return model


def apply_single_device_units(model: nn.Module, param_dtype: torch.dtype, reduce_dtype: torch.dtype):
    """One GPU, no data parallelism: still use the unit machinery (fp32 master + bf16 compute
    copy in flat buffers, fused optimizer), with a shard world of one and no collectives."""
    mp = MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype)
    kw = dict(mesh=None, mp_policy=mp, reshard_after_forward=False)
    if getattr(model, "tok_embeddings", None) is not None:
        fully_shard(model.tok_embeddings, **kw)
    for block in model.layers.values():
        fully_shard(block, **kw)
    if getattr(model, "norm", None) is not None and getattr(model, "output", None) is not None:
        fully_shard([model.norm, model.output], **kw)
    fully_shard(model, **kw)
    return model
