"""Distributed helpers: process-group start-up, determinism, scalar reductions, gradient
clipping, train context.

Parity: torchtitan/distributed/utils.py:30-543 -- ``dist_sum/max/mean`` (:30-58),
``set_determinism`` (one seed broadcast from rank 0, made distinct per pipeline stage;
deterministic algorithm switches, :92-207), ``init_distributed`` (NCCL or ``cuda:nccl,cpu:gloo``
with Flight-Recorder environment, fake backend for dry runs, :251-363), ``set_pg_timeouts``
(:366-394), ``clip_grad_norm_`` (total norm over sharded gradients, extra reduction over
pipeline stages, :397-543), ``maybe_enable_amp`` (:228-248).
"""

from __future__ import annotations

import contextlib
from collections.abc import Callable
import math
import os
from datetime import timedelta

import torch
import torch.distributed as dist
from torch.distributed.tensor import DTensor

from torchtitan_b200.tools.logging import logger
from torchtitan_b200.tools.utils import device_module, device_type

__all__ = [
    "dist_sum", "dist_max", "dist_mean", "set_determinism", "seed_dtensor_rng", "init_distributed", "set_pg_timeouts",
    "clip_grad_norm_", "maybe_enable_amp", "get_train_context", "create_context_parallel_ctx",
]


def _reduce(x, op, mesh, extra=None) -> float:
    if isinstance(x, DTensor):
        x = x.full_tensor()
    x = x.detach().clone().float()
    if mesh is not None:
        dist.all_reduce(x, op=op, group=mesh.get_group() if hasattr(mesh, "get_group") else mesh)
    if extra is not None:
        dist.all_reduce(x, op=op, group=extra.get_group())
    return x.item()


def dist_sum(x: torch.Tensor, mesh, extra_pg=None) -> float:
    return _reduce(x, dist.ReduceOp.SUM, mesh, extra_pg)


def dist_max(x: torch.Tensor, mesh, extra_pg=None) -> float:
    return _reduce(x, dist.ReduceOp.MAX, mesh, extra_pg)


def dist_mean(x: torch.Tensor, mesh, extra_pg=None) -> float:
    n = (mesh.size() if mesh is not None else 1) * (extra_pg.size() if extra_pg is not None else 1)
    return _reduce(x, dist.ReduceOp.SUM, mesh, extra_pg) / n


def set_determinism(parallel_dims, device: torch.device, debug_config, distinct_seed_mesh_dims: list[str] | None = None) -> int:
    """Same seed on all ranks except along ``distinct_seed_mesh_dims`` (default: pipeline). Returns the job's base seed
    (the value every rank shares, before the per-dimension offsets)."""
    distinct_seed_mesh_dims = ["pp"] if distinct_seed_mesh_dims is None else distinct_seed_mesh_dims
    if debug_config.deterministic:
        logger.info("Deterministic algorithm enabled (expect perf degradation).")
        torch.use_deterministic_algorithms(True, warn_only=debug_config.deterministic_warn_only)
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
        os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":4096:8"
    if debug_config.detect_anomaly:
        torch.autograd.set_detect_anomaly(True, check_nan=False)
    seed = debug_config.seed
    world = parallel_dims.world_size
    if seed is None:
        t = torch.get_rng_state()[:8].to(device) if world > 1 and dist.is_initialized() else torch.get_rng_state()[:8]
        if world > 1 and dist.is_initialized():
            dist.broadcast(t, src=0)
        seed = int(t.to("cpu").view(torch.uint64).item() % (2**63))
    base_seed = seed
    rank = dist.get_rank() if dist.is_initialized() else 0
    offset = 0
    mult = 1
    for name in (distinct_seed_mesh_dims if world > 1 else ()):
        if hasattr(parallel_dims, "dim_size"):
            size = parallel_dims.dim_size(name)
            coord = parallel_dims.coordinate(name, rank) if size > 1 else 0
        else:                                   # any object with the mesh accessors of ParallelDims
            mesh = parallel_dims.get_optional_mesh(name)
            size = mesh.size() if mesh is not None else 1
            coord = mesh.get_local_rank() if mesh is not None else 0
        if size > 1:
            offset += coord * mult
            mult *= size
    seed = (seed + offset) % 2**64
    logger.debug(f"rank {rank}: seed {seed}")
    torch.manual_seed(seed)
    os.environ["PYTHONHASHSEED"] = str(seed % 2**32)
    if world > 1 and dist.is_initialized() and torch.device(device).type == "cuda":
        try:
            seed_dtensor_rng(parallel_dims.world_mesh, seed)
        except Exception as e:      # every rank of the job is here, so DTensor's own lazy start-up sync also works
            logger.warning(f"DTensor RNG tracker not pre-seeded ({type(e).__name__}: {e}); falling back to its start-up sync")
    return base_seed


def seed_dtensor_rng(mesh, seed: int) -> None:
    """Create DTensor's random-number tracker for ``mesh`` with ``seed`` and WITHOUT its start-up broadcast.

    The first random op on a DTensor otherwise builds the tracker with a broadcast of rank 0's generator state over the
    default process group. When the mesh covers only part of the job (trainer ranks beside generator ranks), the other
    ranks never enter that broadcast and it pairs up with whatever collective they issue next. Every rank of ``mesh``
    must pass the same ``seed`` (ranks that differ along a pipeline dimension pass their own). A mesh on the CPU has no
    tracker and needs none.
    """
    import torch.distributed.tensor._random as dtensor_random

    if mesh is None or mesh.device_type != "cuda":
        return
    dtensor_random.manual_seed(seed % 2**63, mesh)


def _flight_recorder_env(comm_config, base_folder: str) -> None:
    def setdefault(k, v):
        if k in os.environ:
            logger.warning(f"ENV[{k}] = {os.environ[k]} will be overridden to {v} based on job config")
        os.environ[k] = v

    setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "3")
    if comm_config.trace_buf_size > 0:
        setdefault("TORCH_FR_BUFFER_SIZE", str(comm_config.trace_buf_size))
        setdefault("TORCH_NCCL_DUMP_ON_TIMEOUT", "1")
        dump_dir = os.path.join(base_folder, comm_config.save_traces_folder)
        os.makedirs(dump_dir, exist_ok=True)
        setdefault("TORCH_FR_DUMP_TEMP_FILE", os.path.join(dump_dir, comm_config.save_traces_file_prefix))


def init_fake_mode(world_size: int, comm_mode: str = "fake_backend") -> int:
    """One process standing in for ``world_size`` ranks: collectives of the ``fake`` backend return at once, so that
    configuration, meshes and parallelisation of a large job can be checked without GPUs. ``local_tensor`` and
    ``fake_backend`` are the same here: the parallel runtimes of this framework keep plain local shards and need no
    tensor mode of their own (torchtitan/distributed/utils.py:251-275)."""
    from torch.testing._internal.distributed.fake_pg import FakeStore

    dist.init_process_group("fake", rank=0, world_size=world_size, store=FakeStore())
    return world_size


def init_distributed(comm_config, enable_cpu_backend: bool = False, base_folder: str = "", ranks: list[int] | None = None) -> int:
    """Start the default process group and return the world size."""
    if comm_config.mode in ("fake_backend", "local_tensor"):
        return init_fake_mode(int(os.environ.get("NGPU", os.environ.get("WORLD_SIZE", "1"))), comm_config.mode)
    if not ("RANK" in os.environ and "WORLD_SIZE" in os.environ):
        # single process without a launcher
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29555")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        os.environ.setdefault("LOCAL_RANK", "0")
    if device_type == "cuda":
        _flight_recorder_env(comm_config, base_folder)
        backend = "cuda:nccl,cpu:gloo" if enable_cpu_backend else "nccl"
    else:
        backend = "gloo"
    kwargs = {}
    if ranks is not None:
        kwargs["_ranks"] = ranks
    dist.init_process_group(backend=backend, timeout=timedelta(seconds=comm_config.init_timeout_seconds), **kwargs)
    return dist.get_world_size()


def set_pg_timeouts(timeout: timedelta, parallel_dims) -> None:
    """Tighten collective timeouts after the first step (all ranks meet at a barrier first)."""
    logger.info(f"Synchronizing and adjusting timeout for all ProcessGroups to {timeout}")
    if device_type == "cuda":
        device_module.synchronize()
    dist.barrier(device_ids=[device_module.current_device()] if device_type == "cuda" else None)
    if device_type == "cuda":
        device_module.synchronize()
    groups = [None] + [g for g in parallel_dims._groups.values() if g is not dist.group.WORLD]
    for g in groups:
        try:
            dist.distributed_c10d._set_pg_timeout(timeout, g)
        except Exception as e:  # gloo groups do not support changing the timeout
            logger.debug(f"could not set timeout on {g}: {e}")


def maybe_enable_amp(parallel_dims, mixed_precision_param: str, dev_type: str):
    """FSDP handles mixed precision itself; without it (DDP / single device) use autocast."""
    if parallel_dims.fsdp_enabled:
        logger.info("Mixed precision training is handled by fully_shard")
        return contextlib.nullcontext()
    if parallel_dims.tp_enabled and not parallel_dims.pp_enabled and dev_type == "cuda":
        from torchtitan_b200.config import TORCH_DTYPE_MAP

        # tensor parallel without data-parallel sharding on a GPU: the model runs on single-device mixed-precision units
        # (bf16 compute copies of fp32 masters); autocast covers the inputs that are still fp32
        logger.info("Mixed precision training is handled by single-device units and AMP")
        return torch.autocast(dev_type, dtype=TORCH_DTYPE_MAP[mixed_precision_param])
    if parallel_dims.tp_enabled or parallel_dims.pp_enabled:
        logger.warning("Mixed precision training with TP or PP is only supported when FSDP/HSDP/CP is enabled.")
        logger.info("Mixed precision training is disabled")
        return contextlib.nullcontext()
    from torchtitan_b200.config import TORCH_DTYPE_MAP

    logger.info("Mixed precision training is handled by AMP")
    return torch.autocast(dev_type, dtype=TORCH_DTYPE_MAP[mixed_precision_param])


#: what :func:`get_train_context` returns: a callable giving the context manager a training step runs under
TrainContext = Callable[..., contextlib.AbstractContextManager]


def get_train_context(enable_loss_parallel: bool):
    """Context factory entered around forward+loss+backward. Loss parallel is applied by the
    vocab-parallel loss op itself in this framework, so the context only carries the flag."""

    @contextlib.contextmanager
    def ctx():
        from torchtitan_b200.parallel import tp as _tp

        prev = _tp.LOSS_PARALLEL.enabled
        _tp.LOSS_PARALLEL.enabled = enable_loss_parallel
        try:
            yield
        finally:
            _tp.LOSS_PARALLEL.enabled = prev

    return ctx


def _local(t):
    return t._local_tensor if isinstance(t, DTensor) else t


@torch.no_grad()
def clip_grad_norm_(parameters, max_norm: float, norm_type: float = 2.0, error_if_nonfinite: bool = False,
                    foreach: bool | None = None, pp_mesh=None, ep_enabled: bool = False,
                    fold_into_optimizer: bool = False) -> torch.Tensor:
    """Clip the global gradient norm of (sharded) parameters; returns the total norm.

    Each rank computes the norm of its *local* shards; partial norms are summed over every mesh
    dimension on which a gradient is sharded (read from the DTensor placements; tagged
    tensor/expert-parallel shards add their groups) and over pipeline stages. FSDP units whose
    gradients all live in the unit's flat shard contribute one sum-of-squares launch, and with
    ``fold_into_optimizer`` the clip coefficient is handed to the flat-shard optimizer as a device
    scalar instead of being multiplied into the gradients (the gradients then stay unscaled).
    """
    from torchtitan_b200.ops import optim_ops

    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return torch.tensor(0.0)
    norm_type = float(norm_type)
    inf = math.isinf(norm_type)
    device = _local(params[0].grad).device

    # ---- split parameters into whole FSDP units (flat path) and loose tensors -------------------
    flat_units, loose = [], []
    if norm_type == 2.0:
        by_unit: dict[int, list] = {}
        for p in params:
            ref = getattr(p, "_tt_unit", None)
            if ref is None or getattr(p, "_extra_norm_groups", None):
                loose.append(p)
            else:
                by_unit.setdefault(id(ref[0]), [ref[0], []])[1].append(p)
        for unit, plist in by_unit.values():
            owned = [q.param for q in unit.params if q.param.requires_grad]
            whole = len(plist) == len(owned) and all(
                _local(q.grad).untyped_storage().data_ptr() == unit.grad_shard_flat.untyped_storage().data_ptr()
                for q in plist
            )
            if whole:
                flat_units.append(unit)
            else:
                loose.extend(plist)
    else:
        loose = params

    group_objs: dict[int, object] = {}
    buckets: dict[tuple, list] = {}

    def add(groups, tensor):
        # the reductions of a bucket run group after group: every rank must walk them in the same order, so keep the
        # order in which the parameter lists them (placements first, then tagged groups) -- never an order by object id
        key = tuple(id(g) for g in groups)
        for g in groups:
            group_objs[id(g)] = g
        buckets.setdefault(key, []).append(tensor)

    for unit in flat_units:
        add([unit.shard_group] if unit.shard_world > 1 else [], unit.grad_shard_flat)
    for p in loose:
        g = p.grad
        groups = []
        if isinstance(g, DTensor):
            for i, pl in enumerate(g.placements):
                if pl.is_shard() or pl.is_partial():
                    groups.append(g.device_mesh.get_group(i))
        groups.extend(getattr(p, "_extra_norm_groups", ()))
        add(groups, _local(g))

    total = torch.zeros((), dtype=torch.float32, device=device)
    for key, grads in buckets.items():
        if inf:
            part = torch.stack([g.abs().max().float() if g.numel() else torch.zeros((), device=device) for g in grads]).max()
        elif norm_type == 2.0:
            part = torch.zeros((), dtype=torch.float32, device=device)
            for g in grads:
                if g.numel():
                    part = part + optim_ops.sumsq(g.reshape(-1) if g.is_contiguous() else g.contiguous().view(-1))
        else:
            terms = [torch.linalg.vector_norm(g.float(), norm_type) ** norm_type for g in grads if g.numel()]
            part = torch.stack(terms).sum() if terms else torch.zeros((), device=device)
        for gid in key:
            dist.all_reduce(part, op=dist.ReduceOp.MAX if inf else dist.ReduceOp.SUM, group=group_objs[gid])
        total = torch.maximum(total, part) if inf else total + part
    if pp_mesh is not None:
        dist.all_reduce(total, op=dist.ReduceOp.MAX if inf else dist.ReduceOp.SUM, group=pp_mesh.get_group())
    total_norm = total if inf else total ** (1.0 / norm_type)
    if error_if_nonfinite and not torch.isfinite(total_norm):
        raise RuntimeError(f"The total norm of order {norm_type} for gradients is non-finite")
    coef = torch.clamp(max_norm / (total_norm + 1e-6), max=1.0)
    for unit in flat_units:
        if fold_into_optimizer:
            unit.pending_grad_scale = coef
        else:
            unit.grad_shard_flat.mul_(coef.to(unit.grad_shard_flat.dtype))
    if fold_into_optimizer and loose:
        # parameters with extra norm groups (expert-parallel shards) are reduced one by one above, but when a unit's
        # parameters are all of that kind and their gradients are the unit's flat gradient shard, the coefficient can
        # still ride into the flat-shard optimizer instead of one scaling pass per gradient
        by_unit: dict[int, list] = {}
        for p in loose:
            ref = getattr(p, "_tt_unit", None)
            if ref is not None:
                by_unit.setdefault(id(ref[0]), [ref[0], []])[1].append(p)
        folded = set()
        for unit, plist in by_unit.values():
            owned = [q.param for q in unit.params if q.param.requires_grad]
            if len(plist) == len(owned) and unit.grad_shard_flat is not None and all(
                    _local(q.grad).untyped_storage().data_ptr() == unit.grad_shard_flat.untyped_storage().data_ptr() for q in plist):
                unit.pending_grad_scale = coef
                folded.update(id(q) for q in plist)
        loose = [p for p in loose if id(p) not in folded]
    seen = set()
    for p in loose:
        g = _local(p.grad)
        key = (g.untyped_storage().data_ptr(), g.storage_offset(), g.numel())
        if key not in seen:
            seen.add(key)
            g.mul_(coef.to(g.dtype))
    return total_norm


def create_context_parallel_ctx(*args, **kwargs):
    raise NotImplementedError("context parallel is applied by parallel.cp.apply_cp_to_attention_module")
