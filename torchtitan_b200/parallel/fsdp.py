"""Sharded data parallel runtime (FSDP / HSDP / DDP) built for B200 nodes.

What it provides is what the reference gets from ``torch.distributed.fsdp.fully_shard``
(torchtitan/models/llama3/parallelize.py:287-405, torchtitan/distributed/fsdp.py:8-32):
per-parameter dim-0 sharding that checkpoints see as ``DTensor(Shard(0))``, bf16 parameters
for compute with fp32 master shards and fp32 gradient reduction, reshard-after-forward,
prefetch, HSDP (extra all-reduce over the replicate dimension), DDP, and gradient division
left off (the loss is already divided by the global token count).

How it is built differs:

* A unit owns flat buffers: the fp32 master **shard** (this rank's ``chunk`` rows of every
  parameter, back to back), its compute-dtype **shadow** (what peers gather from; the fused
  optimizer refreshes it in the same launch that updates the master), the gathered
  **unsharded** buffer where each parameter is contiguous, and the fp32 **gradient shard**.
  Optimizer state uses the shard layout too, so AdamW and the gradient norm are one launch
  per unit instead of one per parameter.
* The gather is the forward of one autograd node per unit and the reduce-scatter is that
  node's backward: it runs exactly when every parameter gradient of the unit exists.
* Collectives go through a :class:`ShardComm`. ``C10dComm`` issues one all-gather /
  reduce-scatter per parameter straight into / out of the parameter-contiguous layout (no
  copy-in/copy-out staging; gloo on CPU, NCCL on GPU). ``parallel/nvlink_comm.py`` replaces it
  inside one NVSwitch domain with kernels that pull peers' bf16 shards over NVLink and reduce
  bf16 gradients in fp32 on the owner (half the wire bytes of an fp32 reduce-scatter, same
  arithmetic).
* Gathers run on a side stream one unit ahead (forward and backward); reduce-scatters run on
  another side stream and are joined once at the end of backward.
"""

from __future__ import annotations

import functools
import math
from dataclasses import dataclass, field
from typing import Callable

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.tensor import DTensor, Replicate, Shard

from torchtitan_b200.ops.wgrad_store import WeightGradStore

__all__ = [
    "MixedPrecisionPolicy",
    "fully_shard",
    "replicate",
    "FSDPUnit",
    "ShardComm",
    "C10dComm",
    "fsdp_units",
    "materialize",
]


@dataclass(frozen=True)
class MixedPrecisionPolicy:
    param_dtype: torch.dtype | None = None
    reduce_dtype: torch.dtype | None = None
    output_dtype: torch.dtype | None = None
    cast_forward_inputs: bool = True


@dataclass
class _P:
    """Book-keeping for one parameter of a unit."""

    sites: list  # [(module, attr)] every place the (possibly tied) parameter is bound
    fqn: str
    param: nn.Parameter  # the sharded DTensor parameter users / optimizers / checkpoints see
    full_shape: torch.Size
    shard_dim: int
    rows: int  # size of the sharded dim
    chunk_rows: int  # ceil(rows / W)
    inner: int  # elements per row of the sharded dim
    local_rows: int
    shard_off: int  # element offset of this rank's chunk in the flat shard buffers
    shard_numel: int  # padded chunk elements
    full_off: int  # element offset of the whole parameter in the unsharded buffer
    full_numel: int
    unsharded: torch.Tensor | None = None
    tp_spec: tuple | None = None  # ("shard"|"replicate", dim, group) when tensor parallel tagged the parameter


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def _contig_stride(shape):
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= max(int(s), 1)
    return tuple(reversed(st))


def dtensor_over(local: torch.Tensor, mesh, placements, shape, stride, keep_device: bool = False) -> DTensor:
    """A DTensor whose local shard is ``local`` itself. ``DTensor.from_local`` moves the shard to the mesh's device type;
    CPU-offloaded shards must stay in host memory under a CUDA mesh, so for them the DTensor is built from its spec."""
    if not keep_device and (local.device.type == mesh.device_type or local.is_meta):
        return DTensor.from_local(local, mesh, placements, run_check=False, shape=shape, stride=stride)
    from torch.distributed.tensor._dtensor_spec import DTensorSpec, TensorMeta

    spec = DTensorSpec(mesh, tuple(placements), tensor_meta=TensorMeta(torch.Size(shape), tuple(stride), local.dtype))
    return DTensor(local, spec, requires_grad=local.requires_grad)


class GradSlot:
    """Where a weight-gradient GEMM may write its result directly (skipping the autograd-owned
    temporary): the fp32 gradient shard itself when the shard world is one, or a bf16 slice of the
    NVLink staging buffer that peers reduce from. The GEMM asks :meth:`begin` whether to
    accumulate and the unit learns through ``written`` that nothing is left to copy."""

    __slots__ = ("tensor", "unit", "index", "staging")

    def __init__(self, tensor, unit, index, staging=False):
        self.tensor, self.unit, self.index, self.staging = tensor, unit, index, staging

    def begin(self) -> bool:
        """True when the GEMM must add to what the slot holds. A staging slot only ever holds the gradient of the
        current backward (the reduce kernel adds earlier micro-batches in the fp32 shard), so it accumulates only for a
        second use of the parameter inside one backward; the fp32 shard itself also accumulates across micro-batches."""
        u = self.unit
        acc = (u._slot_accumulate and not self.staging) or u._slot_written[self.index]
        u._slot_written[self.index] = True
        return acc


class ShardComm:
    """Transport used by a unit; the unit handles streams and ordering."""

    def all_gather(self, unit: "FSDPUnit") -> None:
        raise NotImplementedError

    def reduce_scatter(self, unit: "FSDPUnit", grads: list, accumulate: bool) -> None:
        raise NotImplementedError


class C10dComm(ShardComm):
    """c10d collectives issued per parameter directly on the parameter-contiguous layout. ``gather_group``: an optional
    second process group over the same ranks used by the all-gathers only."""

    def __init__(self, gather_group=None):
        self.gather_group = gather_group

    def all_gather(self, unit):
        W, g = unit.shard_world, self.gather_group or unit.shard_group
        src_flat = unit.gather_source()
        works = []
        for p in unit.params:
            n = p.chunk_rows * p.inner
            inp = src_flat[p.shard_off : p.shard_off + n]
            if W == 1:
                unit.unsharded_flat[p.full_off : p.full_off + n].copy_(inp)
            elif p.shard_dim == 0:
                out = unit.unsharded_flat[p.full_off : p.full_off + W * n]
                works.append(dist.all_gather_into_tensor(out, inp, group=g, async_op=True))
            else:
                tmp = torch.empty(W * n, dtype=inp.dtype, device=inp.device)
                dist.all_gather_into_tensor(tmp, inp, group=g)
                unit.place_strided(p, tmp)
        for w in works:
            w.wait()

    def reduce_scatter(self, unit, grads, accumulate):
        W, g, rd = unit.shard_world, unit.shard_group, unit.reduce_dtype
        pending = []
        for i, (p, gr) in enumerate(zip(unit.params, grads)):
            n = p.chunk_rows * p.inner
            dst = unit.grad_shard_flat[p.shard_off : p.shard_off + n]
            if unit.slot_was_written(i):
                # the weight-gradient GEMM wrote (or accumulated) straight into the shard; what autograd
                # delivered is a zero-stride placeholder unless the parameter had another use (tied weights)
                if gr is not None and any(st != 0 for st in gr.stride()):
                    _store(dst, gr.reshape(-1), True)
                continue
            if gr is None:
                if not accumulate:
                    dst.zero_()
                continue
            if W == 1 and unit.replicate_group is None:
                _store(dst, gr.reshape(-1), accumulate)  # one fused cast-copy
                continue
            full = unit.pack_grad(p, gr, rd)  # [W * n], reduce dtype, chunk-major
            if W == 1:
                pending.append((None, dst, full))
            else:
                tmp = torch.empty(n, dtype=rd, device=full.device)
                pending.append((dist.reduce_scatter_tensor(tmp, full, group=g, async_op=True), dst, tmp, full))
        for item in pending:
            work, dst, red = item[0], item[1], item[2]
            if work is not None:
                work.wait()
            if unit.replicate_group is not None:
                dist.all_reduce(red, group=unit.replicate_group)
            _store(dst, red, accumulate)


def _store(dst: torch.Tensor, src: torch.Tensor, accumulate: bool) -> None:
    """``dst (+)= src``; with offloaded shards ``dst`` is pinned host memory and ``src`` comes off the device first."""
    if src.device != dst.device:
        src = src.to(dst.device, dtype=dst.dtype)
    if accumulate:
        dst.add_(src)
    else:
        dst.copy_(src)


class _Streams:
    """Side streams shared by all units of a process (CUDA only)."""

    _inst = None

    def __init__(self, device):
        self.gather = torch.cuda.Stream(device=device, priority=-1)
        self.reduce = torch.cuda.Stream(device=device, priority=-1)

    @classmethod
    def get(cls, device):
        if cls._inst is None:
            cls._inst = _Streams(device)
        return cls._inst


class _UnitGather(torch.autograd.Function):
    """forward: hand out the gathered parameters; backward: reduce-scatter their gradients."""

    @staticmethod
    def forward(ctx, unit, anchor):
        ctx.unit = unit
        if WeightGradStore.enabled:
            ctx.set_materialize_grads(False)      # a parked weight gradient arrives later, not as a tensor of zeros now
        outs = tuple(p.unsharded.view_as(p.unsharded) for p in unit.params)
        frozen = [o for o, p in zip(outs, unit.params) if not p.param.requires_grad]
        if frozen:
            ctx.mark_non_differentiable(*frozen)
        return outs

    @staticmethod
    def backward(ctx, *grads):
        if WeightGradStore.collecting():
            ctx.unit._park_post_backward(list(grads))
        else:
            ctx.unit._post_backward(list(grads))
        return None, None


class FSDPUnit:
    def __init__(self, modules: list[nn.Module], named: list, *, shard_mesh, replicate_mesh, mesh,
                 mp_policy: MixedPrecisionPolicy, reshard_after_forward: bool,
                 shard_placement_fn: Callable | None = None, comm: ShardComm | None = None,
                 compute_device: torch.device | None = None):
        self.modules = modules
        # CPU offload: the sharded parameters, their gradients and (through them) the optimizer state live in host memory;
        # ``compute_device`` holds the compute-dtype copy of the shard that the all-gather reads, the gathered parameters
        # and all activations. None = parameters live where they compute.
        self.compute_device = torch.device(compute_device) if compute_device is not None else None
        self.mp = mp_policy
        self.reshard_after_forward = reshard_after_forward
        self.mesh, self.shard_mesh, self.replicate_mesh = mesh, shard_mesh, replicate_mesh
        if shard_mesh is not None:
            self.shard_group = shard_mesh.get_group()
            self.shard_world = shard_mesh.size()
            self.shard_rank = shard_mesh.get_local_rank()
        else:
            self.shard_group, self.shard_world, self.shard_rank = None, 1, 0
        self.replicate_group = replicate_mesh.get_group() if replicate_mesh is not None else None
        self.comm = comm or C10dComm()
        W, r = self.shard_world, self.shard_rank
        self.params: list[_P] = []
        s_off = f_off = 0
        for sites, fqn, param in named:
            if isinstance(param, DTensor):
                raise NotImplementedError(
                    f"{fqn}: already a DTensor; tensor/expert parallel shards must stay plain local tensors "
                    "before fully_shard (see parallel/tp.py)"
                )
            shape = param.shape
            dim = 0
            if shard_placement_fn is not None and len(shape):
                pl = shard_placement_fn(param)
                if pl is not None:
                    dim = pl.dim
            rows = shape[dim] if len(shape) else 1
            inner = shape.numel() // max(rows, 1) if len(shape) else 1
            chunk = -(-rows // W)
            local_rows = max(0, min(chunk, rows - r * chunk))
            sn = _round_up(chunk * inner, 8)
            fn = _round_up(W * chunk * inner, 8)
            if len(shape) == 0:
                local = param.detach().clone() if param.device.type != "meta" else torch.empty((), dtype=param.dtype, device="meta")
                local_pl = Replicate()
            else:
                lshape = list(shape)
                lshape[dim] = local_rows
                local = torch.empty(lshape, dtype=param.dtype, device=param.device)
                if param.device.type != "meta" and local_rows > 0:
                    local.copy_(param.detach().narrow(dim, r * chunk, local_rows))
                local_pl = Shard(dim) if shard_mesh is not None else Replicate()
            if mesh is None:
                new_param = nn.Parameter(local, requires_grad=param.requires_grad)
            else:
                placements = [local_pl] if mesh.ndim == 1 else [Replicate(), local_pl]
                dt = dtensor_over(local, mesh, placements, shape, _contig_stride(shape))
                new_param = nn.Parameter(dt, requires_grad=param.requires_grad)
            for k, v in param.__dict__.items():  # carry user annotations (e.g. TP placement tags)
                if not k.startswith("__") and k not in ("_local_tensor", "_spec"):
                    try:
                        setattr(new_param, k, v)
                    except Exception:
                        pass
            for m, attr in sites:
                m._parameters[attr] = new_param
            tp_pl = getattr(param, "_tp_placement", None)
            tp_spec = (tp_pl[0], tp_pl[1], getattr(param, "_tp_group", None)) if tp_pl is not None else None
            self.params.append(_P(sites, fqn, new_param, shape, dim, rows, chunk, inner, local_rows,
                                  s_off, sn, f_off, fn, tp_spec=tp_spec))
            s_off += sn
            f_off += fn
        self.shard_numel, self.unsharded_numel = s_off, f_off
        self.orig_dtype = named[0][2].dtype if named else torch.float32
        self.param_dtype = mp_policy.param_dtype or self.orig_dtype
        self.reduce_dtype = mp_policy.reduce_dtype or self.param_dtype
        self.shard_flat = self.shadow_flat = self.grad_shard_flat = self.unsharded_flat = None
        self._anchor = None
        self._gathered = False
        self._gather_event = None
        self._reduce_event = None
        self._keepalive = None
        self._in_backward = False
        self._forward_active = False
        self._shadow_stale = True
        self._materialized = False
        self._grad_dtensors: list = []
        self._fwd_params = None
        self.params_version = 0  # bumped (in lockstep on all ranks) whenever the master shard changes
        self._slots: list = []
        self._wgrad_box: dict | None = None      # parked weight gradients of the backward pass in progress (index -> tensor)
        self._slot_written: list = []
        self._slot_accumulate = False
        self.is_root = False
        self.prefetch_depth = 1  # units gathered ahead of the one that computes (forward: next, backward: prev)
        self.prev: FSDPUnit | None = None
        self.next: FSDPUnit | None = None
        modules[0].register_forward_pre_hook(self._pre_forward, with_kwargs=True, prepend=True)
        modules[-1].register_forward_hook(self._post_forward, prepend=False)

    # ------------------------------------------------------------------ buffers
    @property
    def device(self):
        """Where the unit computes (and gathers)."""
        if self.compute_device is not None:
            return self.compute_device
        return self.storage_device

    @property
    def storage_device(self):
        """Where the sharded parameters live."""
        return self._local(self.params[0].param).device if self.params else torch.device("cpu")

    @property
    def offloaded(self) -> bool:
        return self.compute_device is not None

    @staticmethod
    def _local(param):
        return param._local_tensor if isinstance(param, DTensor) else param.data

    @property
    def uses_cuda(self) -> bool:
        return self.device.type == "cuda"

    def materialize(self) -> None:
        """Move the (now real) sharded parameters into the unit's flat buffers. Runs after
        ``to_empty`` + ``init_weights`` and before the optimizer looks at parameter storage."""
        if self._materialized:
            return
        self._materialized = True
        if not self.params:
            return
        # nn.Module.to_empty() may have replaced plain Parameters by new objects: re-read them
        for p in self.params:
            m, attr = p.sites[0]
            cur = m._parameters[attr]
            if cur is not p.param:
                p.param = cur
                for m2, a2 in p.sites[1:]:
                    m2._parameters[a2] = cur
        dev = self.device
        assert dev.type != "meta", "materialize() needs real parameters (call to_empty/init_weights first)"
        self.shard_flat = self.alloc_shard_buffer(self.orig_dtype, kind="master")
        self.grad_shard_flat = self.alloc_shard_buffer(self.orig_dtype, kind="grad")
        for p in self.params:
            view = self._shard_view(self.shard_flat, p)
            view.copy_(self._local(p.param))
            if isinstance(p.param, DTensor):
                p.param._local_tensor = view
            else:
                p.param.data = view
        if self.param_dtype != self.orig_dtype or self.offloaded:
            self.shadow_flat = self.alloc_shard_buffer(self.param_dtype, kind="shadow")
        for i, p in enumerate(self.params):
            p.param._tt_unit = (self, i)
        self._anchor = torch.zeros((), device=dev, requires_grad=True)
        self._grad_dtensors = [None] * len(self.params)
        self._shadow_stale = True
        self._build_grad_slots()

    def _build_grad_slots(self):
        """Direct weight-gradient destinations for 2-D parameters on CUDA (see GradSlot)."""
        self._slots = [None] * len(self.params)
        self._slot_written = [False] * len(self.params)
        if not self.uses_cuda or self.offloaded:      # a GEMM cannot write into a host-resident gradient shard
            return
        make = getattr(self.comm, "make_grad_slot", None)
        for i, p in enumerate(self.params):
            if len(p.full_shape) != 2 or p.shard_dim != 0 or not p.param.requires_grad:
                continue
            t, staging = None, False
            if make is not None:
                t, staging = make(self, p), True
            elif self.shard_world == 1 and self.replicate_group is None and self.grad_shard_flat.dtype == torch.float32:
                t = self._shard_view(self.grad_shard_flat, p)
            if t is not None:
                self._slots[i] = GradSlot(t, self, i, staging)

    def alloc_shard_buffer(self, dtype, kind: str):
        if self.offloaded and kind in ("master", "grad"):
            buf = torch.zeros(self.shard_numel, dtype=dtype, device="cpu")
            return buf.pin_memory() if torch.cuda.is_available() else buf
        alloc = getattr(self.comm, "alloc_shard_buffer", None)
        if alloc is not None:
            buf = alloc(self, dtype, kind)
            if buf is not None:
                return buf
        return torch.zeros(self.shard_numel, dtype=dtype, device=self.device)

    def _shard_view(self, flat, p: _P):
        if len(p.full_shape) == 0:
            return flat[p.shard_off : p.shard_off + 1].view(())
        shape = list(p.full_shape)
        shape[p.shard_dim] = p.local_rows
        return flat[p.shard_off : p.shard_off + math.prod(shape)].view(shape)

    def gather_source(self):
        """Flat buffer that peers read: the compute-dtype shadow of the master shard."""
        if self.shadow_flat is None:
            return self.shard_flat
        if self._shadow_stale:
            self.shadow_flat.copy_(self.shard_flat, non_blocking=True)      # with offload: pinned host -> device, cast on the way
            self._shadow_stale = False
        return self.shadow_flat

    def mark_params_updated(self, shadow_is_fresh: bool = False) -> None:
        """The optimizer (or a checkpoint load) changed the master shard."""
        self._shadow_stale = not shadow_is_fresh
        self._gathered = False
        self.params_version += 1

    def _storage_alive(self) -> bool:
        return self.unsharded_flat is not None and self.unsharded_flat.untyped_storage().size() > 0

    @property
    def aliases_shard(self) -> bool:
        """With a shard world of one the gathered parameters are the compute-dtype shard itself."""
        return self.shard_world == 1 and all(p.shard_dim == 0 for p in self.params)

    def _alloc_unsharded(self):
        if self.aliases_shard:
            src = self.gather_source()
            if self.unsharded_flat is None or self.unsharded_flat.data_ptr() != src.data_ptr():
                self.unsharded_flat = src
                for p in self.params:
                    p.unsharded = self._full_view(p)
            return
        if self.unsharded_flat is None:
            alloc = getattr(self.comm, "alloc_unsharded_buffer", None)
            buf = alloc(self) if alloc is not None else None
            self.unsharded_flat = buf if buf is not None else torch.empty(
                self.unsharded_numel, dtype=self.param_dtype, device=self.device)
            for p in self.params:
                p.unsharded = self._full_view(p)
        elif not self._storage_alive():
            self.unsharded_flat.untyped_storage().resize_(self.unsharded_numel * self.unsharded_flat.element_size())

    def _full_view(self, p: _P):
        if len(p.full_shape) == 0:
            return self.unsharded_flat[p.full_off : p.full_off + 1].view(())
        return self.unsharded_flat[p.full_off : p.full_off + p.full_shape.numel()].view(p.full_shape)

    def place_strided(self, p: _P, gathered: torch.Tensor):
        """Sharding on a dim other than 0: ``gathered`` is chunk-major; rebuild the tensor."""
        shape = list(p.full_shape)
        shape[p.shard_dim] = p.chunk_rows
        parts = gathered.view(self.shard_world, *shape)
        full = torch.cat(list(parts.unbind(0)), dim=p.shard_dim).narrow(p.shard_dim, 0, p.rows)
        self._full_view(p).copy_(full)

    def pack_grad(self, p: _P, g: torch.Tensor, dtype) -> torch.Tensor:
        """Gradient of a whole parameter -> flat ``[W * chunk * inner]`` in ``dtype``."""
        W, n = self.shard_world, p.chunk_rows * p.inner
        if len(p.full_shape) == 0:
            # a 0-dim parameter is replicated: every rank's chunk receives the sum over ranks
            return g.reshape(1).to(dtype).repeat(W)
        if p.shard_dim == 0:
            if p.rows == W * p.chunk_rows:
                return g.reshape(-1).to(dtype)
            out = torch.zeros(W * n, dtype=dtype, device=g.device)
            out[: p.rows * p.inner].copy_(g.reshape(-1))
            return out
        pad = W * p.chunk_rows - p.rows
        if pad:
            shp = list(g.shape)
            shp[p.shard_dim] = pad
            g = torch.cat((g, g.new_zeros(shp)), dim=p.shard_dim)
        return torch.cat([c.reshape(-1) for c in g.chunk(W, dim=p.shard_dim)]).to(dtype)

    # ------------------------------------------------------------------ gather / free
    def unshard(self, *, async_op: bool = False) -> None:
        """Start (and unless ``async_op`` finish) the gather of this unit's parameters."""
        if not self._materialized:
            self.materialize()
        if not self.params:
            return
        if self.aliases_shard:
            with torch.no_grad():
                first = self.unsharded_flat is None
                if first or self._shadow_stale:
                    if first:
                        self._alloc_unsharded()
                    with torch.autograd._unsafe_preserve_version_counter(self.unsharded_flat):
                        self.gather_source()  # refreshes the shadow in place when it is stale
            self._gathered = True
            return
        if not (self._gathered and self._storage_alive()):
            self._alloc_unsharded()
            with torch.no_grad(), torch.autograd._unsafe_preserve_version_counter(self.unsharded_flat):
                if self.uses_cuda:
                    st = _Streams.get(self.device)
                    st.gather.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(st.gather):
                        self.comm.all_gather(self)
                        self._gather_event = st.gather.record_event()
                else:
                    self.comm.all_gather(self)
            self._gathered = True
        if not async_op and self._gather_event is not None:
            torch.cuda.current_stream().wait_event(self._gather_event)
            self._gather_event = None

    def reshard(self) -> None:
        if self.aliases_shard:
            return
        if self._storage_alive():
            if self.uses_cuda:
                # the side stream may still be writing a prefetched gather
                if self._gather_event is not None:
                    torch.cuda.current_stream().wait_event(self._gather_event)
                    self._gather_event = None
            self.unsharded_flat.untyped_storage().resize_(0)
        self._gathered = False

    def _bind(self, tensors):
        for p, t in zip(self.params, tensors):
            for m, attr in p.sites:
                m._parameters[attr] = t

    def _bind_sharded(self):
        for p in self.params:
            for m, attr in p.sites:
                m._parameters[attr] = p.param

    # ------------------------------------------------------------------ hooks
    def _needs_grad(self) -> bool:
        return torch.is_grad_enabled() and any(p.param.requires_grad for p in self.params)

    def _pre_forward(self, module, args, kwargs):
        cast_result = None
        if self.is_root and self.mp.cast_forward_inputs and self.mp.param_dtype is not None:
            dt = self.mp.param_dtype
            cast = lambda t: t.to(dt) if torch.is_tensor(t) and t.is_floating_point() else t
            cast_result = tuple(cast(a) for a in args), {k: cast(v) for k, v in kwargs.items()}
        if self._in_backward or self._forward_active or not self.params:
            return cast_result  # recompute inside backward, a re-entrant call, or nothing to gather
        self._forward_active = True
        self.unshard()
        ahead = self.next
        for _ in range(max(self.prefetch_depth, 1)):
            if ahead is None or ahead._in_backward:
                break
            ahead.unshard(async_op=True)
            ahead = ahead.next
        if self._needs_grad():
            outs = _UnitGather.apply(self, self._anchor)
        else:
            outs = tuple(p.unsharded for p in self.params)
        # the same tensor objects are re-bound for recompute in backward; with several forwards in flight before the
        # first backward (pipeline micro-batches) each backward needs ITS forward's tensors, so the output hooks carry them
        self._fwd_params = outs
        if WeightGradStore.enabled:
            # split backward steps (zero-bubble pipeline schedules): linear layers park their weight-gradient GEMMs and
            # hand the result to this unit later, see _park_post_backward. Gradient slots are not used then: several
            # micro-batches can be between their two halves at once and would share one staging buffer
            if self._needs_grad():
                for i, o in enumerate(outs):
                    o._wgrad_sink = (self, i)
        elif self._slots:
            for o, slot in zip(outs, self._slots):
                if slot is not None:
                    o._grad_slot = slot
        self._bind(outs)
        return cast_result

    def _post_forward(self, module, args, output):
        if self._in_backward or not self._forward_active:
            return output
        self._forward_active = False
        self._bind_sharded()
        if self._needs_grad():
            self._hook_outputs(output, self._fwd_params)
        if self.reshard_after_forward:
            self.reshard()
        if self.mp.output_dtype is not None and torch.is_tensor(output):
            output = output.to(self.mp.output_dtype)
        return output

    def _hook_outputs(self, output, fwd_params):
        hook = functools.partial(self._pre_backward, fwd_params)

        def visit(o):
            if torch.is_tensor(o):
                if o.requires_grad:
                    o.register_hook(hook)
            elif isinstance(o, (list, tuple)):
                for x in o:
                    visit(x)
            elif isinstance(o, dict):
                for x in o.values():
                    visit(x)

        visit(output)

    def _pre_backward(self, fwd_params, grad):
        if not self._in_backward:
            self._in_backward = True
            first = next((p for p in self.params if p.param.requires_grad), None)
            self._slot_accumulate = first is not None and first.param.grad is not None
            self._slot_written = [False] * len(self.params)
            guard = getattr(self.comm, "before_grad_writes", None)
            if guard is not None:
                guard(self)  # peers may still be reading the staging buffer of the previous micro-batch
            self.unshard()
            behind = self.prev
            for _ in range(max(self.prefetch_depth, 1)):
                if behind is None or not behind.reshard_after_forward or behind._in_backward:
                    break
                behind.unshard(async_op=True)
                behind = behind.prev
            self._bind(fwd_params if fwd_params is not None else tuple(p.unsharded for p in self.params))
            _BackwardEnd.register(self)
        return grad

    def wgrad_box(self) -> dict:
        """Where the parked weight-gradient closures of the backward pass in progress put their results."""
        if self._wgrad_box is None:
            self._wgrad_box = {}
        return self._wgrad_box

    def _park_post_backward(self, grads):
        """Input-gradient half of a split backward step: keep what autograd delivered (norm weights, biases, everything
        that is not a parked linear weight), leave backward mode, and queue the reduction behind the parked GEMMs of this
        pass; the weight-gradient half runs the queue in order, so the reduction sees the complete set."""
        box, self._wgrad_box = self.wgrad_box(), None

        def reduce_parked(unit=self, grads=grads, box=box):
            for i, gw in box.items():
                grads[i] = gw if grads[i] is None else grads[i] + gw.to(grads[i].dtype)
            box.clear()
            guard = getattr(unit.comm, "before_grad_writes", None)
            if guard is not None:
                guard(unit)          # a reduction of another micro-batch may have run since this pass entered backward
            unit._reduce_grads(grads)
            unit.wait_for_reduce()

        WeightGradStore.put(reduce_parked)
        self._finish_backward()

    def _post_backward(self, grads):
        self._reduce_grads(grads)
        self._finish_backward()

    def _reduce_grads(self, grads):
        # parameters replicated over tensor parallel saw only a sequence shard: sum their gradients
        for i, p in enumerate(self.params):
            if p.tp_spec is not None and p.tp_spec[0] == "replicate" and grads[i] is not None:
                g = grads[i] if grads[i].is_contiguous() else grads[i].contiguous()
                dist.all_reduce(g, group=p.tp_spec[2])
                grads[i] = g
        first = next((p for p in self.params if p.param.requires_grad), None)
        accumulate = first is not None and first.param.grad is not None
        with torch.no_grad():
            if self.uses_cuda:
                st = _Streams.get(self.device)
                st.reduce.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(st.reduce):
                    self.comm.reduce_scatter(self, grads, accumulate)
                    self._reduce_event = st.reduce.record_event()
                self._keepalive = grads
            else:
                self.comm.reduce_scatter(self, grads, accumulate)
        for i, p in enumerate(self.params):
            if p.param.requires_grad and p.param.grad is None:
                p.param.grad = self._grad_view(i)

    def _finish_backward(self):
        self._in_backward = False
        self._forward_active = False
        self._fwd_params = None
        self._slot_written = [False] * len(self.params)
        self._bind_sharded()
        if self.reshard_after_forward:
            self.reshard()

    def slot_was_written(self, i: int) -> bool:
        return bool(self._slots) and self._slots[i] is not None and self._slot_written[i]

    def wait_for_reduce(self):
        if self._reduce_event is not None:
            torch.cuda.current_stream().wait_event(self._reduce_event)
            self._reduce_event = None
        self._keepalive = None

    def _grad_view(self, i: int):
        if self._grad_dtensors[i] is None:
            p = self.params[i]
            local = self._shard_view(self.grad_shard_flat, p)
            if isinstance(p.param, DTensor):
                self._grad_dtensors[i] = dtensor_over(local, self.mesh, p.param.placements, p.full_shape,
                                                      _contig_stride(p.full_shape))
            else:
                self._grad_dtensors[i] = local
        return self._grad_dtensors[i]


class _BackwardEnd:
    """Runs once per backward pass after autograd is done: joins the reduce stream and lets
    units whose gather node never ran (unused parameters) leave backward mode."""

    _pending: list = []
    _queued = False

    @classmethod
    def register(cls, unit):
        cls._pending.append(unit)
        if not cls._queued:
            cls._queued = True
            torch.autograd.Variable._execution_engine.queue_callback(cls._run)

    @classmethod
    def _run(cls):
        units, cls._pending, cls._queued = cls._pending, [], False
        for u in units:
            if u._in_backward:
                if WeightGradStore.collecting() and u._wgrad_box is not None:
                    # every gradient of the unit was parked (a unit of bias-free linear layers): its gather node had
                    # nothing to run on, the reduction still has to follow the parked GEMMs
                    u._park_post_backward([None] * len(u.params))
                else:
                    u._finish_backward()
            u.wait_for_reduce()


# ---------------------------------------------------------------------- public API
def _managed_params(modules: list[nn.Module]):
    """Unique parameters not owned by a nested unit: [(sites, fqn, param)]."""
    order, by_id = [], {}

    def walk(m: nn.Module, prefix: str, top: bool):
        if not top and getattr(m, "_fsdp_unit", None) is not None:
            return
        for name, p in m._parameters.items():
            if p is None:
                continue
            if id(p) in by_id:
                by_id[id(p)][0].append((m, name))
            else:
                by_id[id(p)] = ([(m, name)], prefix + name, p)
                order.append(id(p))
        for cname, child in m._modules.items():
            if child is not None:
                walk(child, f"{prefix}{cname}.", False)

    for i, mod in enumerate(modules):
        walk(mod, "" if len(modules) == 1 else f"[{i}].", True)
    return [by_id[i] for i in order]


def _split_mesh(mesh):
    if mesh is None:
        return None, None
    if mesh.ndim == 2:
        names = mesh.mesh_dim_names
        return mesh[names[0]], mesh[names[1]]
    return None, mesh


def fully_shard(module, *, mesh, mp_policy: MixedPrecisionPolicy | None = None,
                reshard_after_forward: bool = True, shard_placement_fn: Callable | None = None,
                offload_policy=None, comm: ShardComm | None = None, compute_device=None):
    """Shard the parameters of ``module`` (a module, or a list of modules executed in list
    order and gathered together) that no nested unit already owns.

    ``mesh``: 1-D ``fsdp`` mesh, or 2-D ``[dp_replicate, fsdp]`` for HSDP.
    """
    if offload_policy is not None and compute_device is None:
        # torch's ``CPUOffloadPolicy()`` spelling: keep shards on the host, compute on the current accelerator
        compute_device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    modules = list(module) if isinstance(module, (list, tuple)) else [module]
    named = _managed_params(modules)
    rep, shard = _split_mesh(mesh)
    unit = FSDPUnit(modules, named, shard_mesh=shard, replicate_mesh=rep, mesh=mesh,
                    mp_policy=mp_policy or MixedPrecisionPolicy(), reshard_after_forward=reshard_after_forward,
                    shard_placement_fn=shard_placement_fn, comm=comm, compute_device=compute_device)
    for m in modules:
        m._fsdp_unit = unit
    return module


def replicate(module, *, mesh, mp_policy: MixedPrecisionPolicy | None = None, comm: ShardComm | None = None):
    """DDP: whole parameters on every rank, gradients all-reduced over the 1-D ``mesh``.

    Same unit machinery with a shard world of one, so bucketing (one flat gradient buffer per
    unit), mixed precision and stream overlap are shared with FSDP.
    """
    modules = list(module) if isinstance(module, (list, tuple)) else [module]
    named = _managed_params(modules)
    unit = FSDPUnit(modules, named, shard_mesh=None, replicate_mesh=mesh, mesh=mesh,
                    mp_policy=mp_policy or MixedPrecisionPolicy(), reshard_after_forward=False, comm=comm)
    for m in modules:
        m._fsdp_unit = unit
    return module


def fsdp_units(model: nn.Module) -> list[FSDPUnit]:
    seen, out = set(), []
    for m in model.modules():
        u = getattr(m, "_fsdp_unit", None)
        if u is not None and id(u) not in seen:
            seen.add(id(u))
            out.append(u)
    return out


def materialize(model: nn.Module) -> None:
    """Finish FSDP set-up once parameters are real: flat buffers + execution-order links."""
    units = fsdp_units(model)
    for u in units:
        u.materialize()
    root = getattr(model, "_fsdp_unit", None)
    if root is not None:
        root.is_root = True
    chain = [u for u in units if u is not root and u.params]
    if root is not None and root.params:
        chain = [root] + chain
    for a, b in zip(chain, chain[1:]):
        a.next, b.prev = b, a
