"""FSDP transport over NVLink peer memory (single NVSwitch domain).

Each rank of the shard group allocates one arena with ``cudaMalloc``, exports it with CUDA IPC
and maps every peer's arena. Per FSDP unit the arena holds the bf16 **shadow shard** (written
by the fused optimizer, read by the peers' all-gather kernel) and the bf16 **gradient staging
buffer** in the gathered layout (written directly by the weight-gradient GEMMs through
``GradSlot``, read by the owners' reduce-scatter kernel), plus two version flags per unit.

* all-gather = one ``tt_allgather_pull`` launch: every parameter chunk of every peer is copied
  straight to its final place in the parameter-contiguous gathered buffer.
* reduce-scatter = one ``tt_reduce_scatter_pull`` launch: this rank's slice of all peers' staging
  buffers is summed in fp32 in rank order and written (or accumulated) into the fp32 gradient
  shard; bf16 crosses NVLink, the arithmetic equals an fp32 reduce of the bf16 gradients.

Cross-rank ordering: a rank publishes ``version`` in its flag after the producing work is
queued on the same stream; consumers spin (bounded) until all flags reach the version they
expect. Write-after-read hazards:

* a shadow shard is only rewritten by the optimizer after every reduce-scatter of the step, which
  needs every peer's backward (hence every peer's gathers) of that step to be done;
* a staging buffer is rewritten by the next backward of its unit. Across optimizer steps the
  all-gather flags order that (a peer's next forward needs this rank's optimizer, which follows
  all of this rank's reduce kernels). Within one optimizer step (gradient accumulation, pipeline
  micro-batches) nothing else does, so every rank publishes a third flag, "my reduce kernel for
  version v has read your staging", and :meth:`NvlinkComm.before_grad_writes` (called when a unit
  enters backward) waits, bounded, for all peers' flags before the first gradient write.

What the reference does for the same step: NCCL all-gather / reduce-scatter with copy-in,
copy-out and fp32 casts around them (``torch.distributed.fsdp``), see
torchtitan/models/llama3/parallelize.py:340-364.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from torchtitan_b200.ops import native
from torchtitan_b200.tools.logging import logger

from .fsdp import FSDPUnit, ShardComm

native.register_optional("tt_ipc_alloc", [ctypes.POINTER(ctypes.c_void_p), ctypes.c_longlong])
native.register_optional("tt_ipc_free", [ctypes.c_void_p])
native.register_optional("tt_ipc_handle_size", [])
native.register_optional("tt_ipc_get_handle", [ctypes.c_void_p, ctypes.c_void_p])
native.register_optional("tt_ipc_open", [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)])
native.register_optional("tt_ipc_close", [ctypes.c_void_p])
native.register_optional("tt_memset", [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p])
native.register_optional("tt_set_flag", [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p])
_PP = ctypes.POINTER(ctypes.c_void_p)
native.register_optional("tt_allgather_pull", [_PP, _PP, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p])
native.register_optional("tt_reduce_scatter_pull", [_PP, _PP, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                                    ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p])
native.register_optional("tt_allreduce_pull_f32", [_PP, _PP, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                                   ctypes.c_void_p])
native.register_optional("tt_comm_error", [ctypes.POINTER(ctypes.c_int)])
native.register_optional("tt_comm_set_wait_ns", [ctypes.c_ulonglong])


class _RawCuda:
    """Zero-copy torch view of raw device memory (through ``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def tensor_from_ptr(ptr: int, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device).view(dtype)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def node_identity() -> int:
    """62-bit number that is the same for all processes of one machine boot and differs between machines."""
    import hashlib
    import socket

    ident = socket.gethostname()
    try:
        with open("/proc/sys/kernel/random/boot_id") as f:
            ident += f.read().strip()
    except OSError:
        pass
    return int.from_bytes(hashlib.md5(ident.encode()).digest()[:8], "little") >> 2


def peer_memory_group_ok(group, extra_ok: bool = True, max_world: int = 16) -> bool:
    """Collective over ``group``: True on every rank when the group can share memory through CUDA IPC, that is when
    ``extra_ok`` holds on every rank, the group has 2..``max_world`` ranks, all of them run on this machine (a job over
    several nodes can have groups of the right size whose ranks sit on different hosts, where the IPC handles mean
    nothing) and this rank's GPU can map every other GPU of the machine. Otherwise False on every rank, and the callers
    keep to the collectives."""
    W = dist.get_world_size(group)
    ok = bool(extra_ok) and 2 <= W <= max_world
    if torch.cuda.is_available():
        me = torch.cuda.current_device()
        ok = ok and torch.cuda.device_count() >= W and all(
            torch.cuda.can_device_access_peer(me, d) for d in range(torch.cuda.device_count()) if d != me)
        device = "cuda"
    else:
        ok, device = False, "cpu"
    return all_ranks_agree_on_one_node(group, ok, device)


def all_ranks_agree_on_one_node(group, ok: bool, device: str) -> bool:
    """One all-reduce: every rank said ``ok`` and every rank reports the same node identity."""
    h = node_identity()
    t = torch.tensor([1 if ok else 0, h, -h], dtype=torch.int64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    t = t.tolist()
    return t[0] == 1 and t[1] == -t[2]


class SymmetricHeap:
    """One IPC-shared arena per rank with a bump allocator that is replayed identically on every
    rank, so an offset names the same object everywhere."""

    FLAG_BYTES = 1 << 16

    def __init__(self, group, nbytes: int, device: torch.device):
        L = native.lib()
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.nbytes = (int(nbytes) + self.FLAG_BYTES + 4095) // 4096 * 4096
        base = ctypes.c_void_p()
        native.check(L.tt_ipc_alloc(ctypes.byref(base), self.nbytes), "tt_ipc_alloc")
        self.base = base.value
        native.check(L.tt_memset(self.base, 0, self.nbytes, _stream()), "tt_memset")
        torch.cuda.synchronize()
        hsize = L.tt_ipc_handle_size()
        buf = ctypes.create_string_buffer(hsize)
        native.check(L.tt_ipc_get_handle(self.base, buf), "tt_ipc_get_handle")
        handles: list = [None] * self.world
        dist.all_gather_object(handles, (bytes(buf.raw), self.nbytes), group=group)
        self.peer_base: list[int] = []
        for r, (h, nb) in enumerate(handles):
            assert nb == self.nbytes, "symmetric heap sizes differ across ranks"
            if r == self.rank:
                self.peer_base.append(self.base)
                continue
            out = ctypes.c_void_p()
            rc = L.tt_ipc_open(ctypes.create_string_buffer(h, hsize), ctypes.byref(out))
            if rc != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle failed for peer {r} (code {rc})")
            self.peer_base.append(out.value)
        self._top = self.FLAG_BYTES  # flags live at the start of the arena
        self._next_flag = 0
        dist.barrier(group=group)

    def alloc(self, nbytes: int, align: int = 256) -> int:
        off = (self._top + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted ({off + nbytes} > {self.nbytes})")
        self._top = off + nbytes
        return off

    def alloc_flag(self) -> int:
        off = self._next_flag * 4
        self._next_flag += 1
        assert off < self.FLAG_BYTES
        return off

    def local_tensor(self, off: int, numel: int, dtype) -> torch.Tensor:
        return tensor_from_ptr(self.base + off, numel, dtype, self.device)

    def peer_ptrs(self, off: int):
        arr = (ctypes.c_void_p * self.world)(*[b + off for b in self.peer_base])
        return ctypes.cast(arr, _PP), arr


class NvlinkComm(ShardComm):
    def __init__(self, mesh, heap_bytes: int):
        shard_mesh = mesh[mesh.mesh_dim_names[-1]] if mesh.ndim == 2 else mesh
        self.group = shard_mesh.get_group()
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.heap = SymmetricHeap(self.group, heap_bytes, self.device)
        self.world, self.rank = self.heap.world, self.heap.rank
        self._units: dict[int, dict] = {}
        logger.info(f"NVLink FSDP transport: {self.world} ranks, {self.heap.nbytes / 2**30:.2f} GiB symmetric heap per rank")

    # ------------------------------------------------------------------ factory
    @classmethod
    def maybe_create(cls, mesh, model=None, param_dtype=torch.bfloat16):
        if not native.available() or mesh is None or param_dtype != torch.bfloat16:
            return None
        shard_mesh = mesh[mesh.mesh_dim_names[-1]] if mesh.ndim == 2 else mesh
        W = shard_mesh.size()
        if W < 2 or W > 16:
            return None
        # all ranks of the group must be GPUs of this process's node with peer access
        if not peer_memory_group_ok(shard_mesh.get_group()):
            logger.info("NVLink FSDP transport unavailable (ranks on several nodes or no peer access); using c10d collectives")
            return None
        # a tied weight is reachable from two wrapped units and each keeps its own flat buffers: count it twice
        nparams = sum(p.numel() for _, p in model.named_parameters(remove_duplicate=False)) if model is not None else 0
        nunits = 4 + (len(model.layers) if model is not None and hasattr(model, "layers") else 64)
        # shadow shard (2 B / W) + staging (2 B) per parameter, rounding slack per unit and per parameter
        heap_bytes = int(2.05 * nparams * (1 + 1.0 / W)) + nunits * (1 << 20) + (64 << 20)
        return cls(mesh, heap_bytes)

    # ------------------------------------------------------------------ per-unit state
    def _state(self, unit: FSDPUnit) -> dict:
        st = self._units.get(id(unit))
        if st is None:
            h = self.heap
            st = {"shadow_off": None, "staging_off": None, "flag_shadow": h.alloc_flag(), "flag_grad": h.alloc_flag(),
                  "flag_done": h.alloc_flag(), "gather_version": 0, "grad_version": 0, "rs_params_version": None, "segs": None}
            self._units[id(unit)] = st
        return st

    def supports(self, unit: FSDPUnit) -> bool:
        return (unit.param_dtype == torch.bfloat16 and unit.orig_dtype == torch.float32 and unit.shard_world == self.world
                and all(p.shard_dim == 0 and len(p.full_shape) > 0 for p in unit.params))

    def alloc_shard_buffer(self, unit: FSDPUnit, dtype, kind: str):
        if kind != "shadow" or not self.supports(unit):
            return None
        st = self._state(unit)
        st["shadow_off"] = self.heap.alloc(unit.shard_numel * 2)
        st["staging_off"] = self.heap.alloc(unit.unsharded_numel * 2)
        st["staging"] = self.heap.local_tensor(st["staging_off"], unit.unsharded_numel, torch.bfloat16)
        segs = torch.tensor([[p.shard_off, p.full_off, p.chunk_rows * p.inner] for p in unit.params], dtype=torch.int64)
        st["segs"] = segs.to(self.device)
        return self.heap.local_tensor(st["shadow_off"], unit.shard_numel, torch.bfloat16)

    def make_grad_slot(self, unit: FSDPUnit, p):
        st = self._units.get(id(unit))
        if st is None or st.get("staging") is None:
            return None
        return st["staging"][p.full_off : p.full_off + p.rows * p.inner].view(p.full_shape)

    # ------------------------------------------------------------------ collectives
    def _fallback(self):
        from .fsdp import C10dComm

        if not hasattr(self, "_c10d"):
            self._c10d = C10dComm()
        return self._c10d

    def all_gather(self, unit: FSDPUnit) -> None:
        st = self._units.get(id(unit))
        if st is None or st.get("shadow_off") is None:
            return self._fallback().all_gather(unit)
        L = native.lib()
        unit.gather_source()  # refresh the shadow from the master shard when it is stale
        version = unit.params_version + 1
        h = self.heap
        native.check(L.tt_set_flag(h.base + st["flag_shadow"], version, _stream()), "tt_set_flag")
        ptrs, keep1 = h.peer_ptrs(st["shadow_off"])
        flags, keep2 = h.peer_ptrs(st["flag_shadow"])
        native.check(L.tt_allgather_pull(ptrs, flags, st["segs"].data_ptr(), len(unit.params), unit.unsharded_flat.data_ptr(),
                                         self.world, self.rank, version, 0, 8, _stream()), "tt_allgather_pull")

    def reduce_scatter(self, unit: FSDPUnit, grads, accumulate: bool) -> None:
        st = self._units.get(id(unit))
        if st is None or st.get("staging") is None:
            return self._fallback().reduce_scatter(unit, grads, accumulate)
        L = native.lib()
        staging = st["staging"]
        for i, (p, g) in enumerate(zip(unit.params, grads)):
            n = p.rows * p.inner if len(p.full_shape) else 1
            view = staging[p.full_off : p.full_off + n]
            if unit.slot_was_written(i):
                if g is not None and any(s != 0 for s in g.stride()):
                    view.add_(g.reshape(-1))
                continue
            if g is None:
                view.zero_()
            else:
                view.copy_(g.reshape(-1))
        st["grad_version"] += 1
        version = st["grad_version"]
        h = self.heap
        native.check(L.tt_set_flag(h.base + st["flag_grad"], version, _stream()), "tt_set_flag")
        ptrs, keep1 = h.peer_ptrs(st["staging_off"])
        flags, keep2 = h.peer_ptrs(st["flag_grad"])
        out = unit.grad_shard_flat
        acc = accumulate
        if unit.replicate_group is not None and accumulate:
            out, acc = torch.empty_like(unit.grad_shard_flat), False
        native.check(L.tt_reduce_scatter_pull(ptrs, flags, st["segs"].data_ptr(), len(unit.params), out.data_ptr(), self.world,
                                              self.rank, version, int(acc), 64, _stream()), "tt_reduce_scatter_pull")
        # "read done": the peers' staging buffers of this version may be overwritten from here on
        native.check(L.tt_set_flag(h.base + st["flag_done"], version, _stream()), "tt_set_flag")
        st["rs_params_version"] = unit.params_version
        if unit.replicate_group is not None:
            dist.all_reduce(out, group=unit.replicate_group)
            if out is not unit.grad_shard_flat:
                unit.grad_shard_flat.add_(out)

    def needs_staging_wait(self, unit: FSDPUnit) -> bool:
        """True when this unit's staging buffer was reduced since the last optimizer step: a peer may still be reading it."""
        st = self._units.get(id(unit))
        return (st is not None and st.get("staging") is not None and st["grad_version"] > 0
                and st["rs_params_version"] == unit.params_version)

    def before_grad_writes(self, unit: FSDPUnit) -> None:
        """Called on the compute stream when ``unit`` enters backward, before any weight-gradient GEMM writes staging.
        Waits (bounded, error word on expiry) until every peer's reduce kernel of the previous micro-batch has read this
        rank's staging buffer. Skipped when an optimizer step lies in between (see the module docstring)."""
        if not self.needs_staging_wait(unit):
            return
        st = self._units[id(unit)]
        flags, keep = self.heap.peer_ptrs(st["flag_done"])
        native.check(native.lib().tt_wait_flags(flags, self.world, st["grad_version"], _stream()), "tt_wait_flags")

    def errors(self):
        out = (ctypes.c_int * 4)()
        code = native.lib().tt_comm_error(out)
        return None if code == 0 else {"code": out[0], "peer": out[1], "expected": out[2], "seen": out[3]}
