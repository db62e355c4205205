"""Policy weight transfer from the trainer's sharded parameters to generator replicas.

The reference gathers every parameter to a full tensor, ships the dict through an RPC and re-distributes
it (torchtitan/experiments/rl/unified/actors/trainer.py:226-239, actors/generator.py:307-335). Here the
generator's parameters live in one flat bf16 *arena* (``ParamArena``); a sync is: each trainer rank
casts its shards into the arena layout, and one collective moves the arena --

* colocated (trainer and generator share a GPU): ``sync_local`` copies/casts trainer parameters
  straight into the arena, shard by shard, with no intermediate full tensors for unsharded ones;
* disaggregated: ``broadcast_arena`` sends the whole arena with a single broadcast over NVLink
  (one launch for all weights instead of one RPC per tensor).

The arena is double-buffered: writes go to the inactive half and ``flip()`` repoints the generator's
parameters, so decoding never observes a half-written model.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn


def full_tensor(p: torch.Tensor) -> torch.Tensor:
    """The unsharded value of a (possibly FSDP-, tensor- or expert-parallel-sharded) parameter: a collective of every
    group the parameter is sharded over."""
    from torchtitan_b200.parallel.global_view import global_view

    v = global_view(p)
    t = v.full_tensor() if hasattr(v, "full_tensor") else v
    return t.detach()


def build_bare_model(model_spec, dtype_name: str, device) -> nn.Module:
    """An uninitialised model in the generator's dtype and layout (no engine, no KV cache): the staging side of a sync."""
    from torchtitan_b200.config import TORCH_DTYPE_MAP

    device = torch.device(device) if device is not None else torch.device(
        f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cpu")
    dtype = TORCH_DTYPE_MAP[dtype_name] if device.type == "cuda" else torch.float32
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device("meta"):
            model = model_spec.model.build()
    finally:
        torch.set_default_dtype(old)
    model.to_empty(device=device)
    with torch.no_grad():
        model.init_weights(buffer_device=device)     # also restores parameter tying, so both sides agree on the layout
    for p in model.parameters():
        p.requires_grad_(False)
    return model


class ParamArena:
    """All parameters of ``model`` re-seated as views of one flat buffer (two halves when double-buffered)."""

    def __init__(self, model: nn.Module, double_buffer: bool = True, alloc=None):
        """``alloc(numel, dtype) -> flat tensor`` lets the halves live in an NVLink-mapped symmetric heap."""
        self.model = model
        params = list(dict(model.named_parameters()).items())
        self.names = [n for n, _ in params]
        self.shapes = [tuple(p.shape) for _, p in params]
        self.offsets, off = [], 0
        for _, p in params:
            self.offsets.append(off)
            off += (p.numel() + 127) // 128 * 128          # 256-byte aligned slices
        self.numel = off
        p0 = params[0][1]
        make = alloc or (lambda n, dt: torch.zeros(n, dtype=dt, device=p0.device))
        self.halves = [make(off, p0.dtype) for _ in range(2 if double_buffer else 1)]
        self.active = 0
        with torch.no_grad():
            for (_, p), o in zip(params, self.offsets):
                self.halves[0][o : o + p.numel()].copy_(p.reshape(-1))
        # tied parameters (one tensor under two names) appear once in named_parameters and stay tied after re-seating
        self._seat(0)

    def _views(self, half: int):
        buf = self.halves[half]
        return [buf[o : o + int(torch.tensor(s).prod()) if s else o + 1].view(s) for o, s in zip(self.offsets, self.shapes)]

    def _seat(self, half: int) -> None:
        named = dict(self.model.named_parameters())
        for n, v in zip(self.names, self._views(half)):
            named[n].data = v
        self.active = half

    @property
    def inactive(self) -> int:
        return (self.active + 1) % len(self.halves)

    def staging(self) -> dict[str, torch.Tensor]:
        """Views of the half that is *not* being read by the generator."""
        return dict(zip(self.names, self._views(self.inactive)))

    def flip(self) -> None:
        self._seat(self.inactive)


@torch.no_grad()
def sync_local(trainer_model: nn.Module, arena: ParamArena) -> int:
    """Cast/copy every trainer parameter into the arena's staging half and flip. Returns bytes written."""
    dst = arena.staging()
    n = 0
    for name, p in trainer_model.named_parameters():
        if name in dst:
            dst[name].copy_(full_tensor(p))
            n += dst[name].numel() * dst[name].element_size()
    arena.flip()
    return n


@torch.no_grad()
def broadcast_arena(arena: ParamArena, src: int, group=None, trainer_model: nn.Module | None = None) -> None:
    """Trainer rank ``src`` fills its arena's staging half from ``trainer_model``; every rank of ``group``
    receives it with one broadcast and flips."""
    if trainer_model is not None:
        dst = arena.staging()
        for name, p in trainer_model.named_parameters():
            if name in dst:
                dst[name].copy_(full_tensor(p))
    dist.broadcast(arena.halves[arena.inactive], src=src, group=group)
    arena.flip()


def arena_layout(model: nn.Module) -> tuple[dict[str, int], int]:
    """(name -> element offset, total elements) of the arena a :class:`ParamArena` would build for ``model`` (works on
    meta tensors: trainer ranks use it to address generator arenas they never allocate)."""
    offsets, off = {}, 0
    for n, p in model.named_parameters():
        offsets[n] = off
        off += (p.numel() + 127) // 128 * 128
    return offsets, off


class NvlinkWeightSync:
    """Peer-memory weight sync: each trainer rank casts the fp32 master shards it owns to bf16 and writes them directly
    into every generator replica's (inactive) arena half with one kernel (``tt_push_cast``), then publishes the version on
    a flag in each generator's heap; a generator waits (stream-ordered, bounded) for all trainer flags and flips.

    All ranks of the job build one symmetric heap; generator arenas are allocated from it on every rank (trainer ranks
    leave theirs unused) so an offset addresses the same arena half everywhere. Trainer parameters must be data-parallel
    sharded on dim 0 by the framework's FSDP runtime (or unsharded); other layouts use the broadcast path."""

    def __init__(self, group, trainer_ranks: list[int], generator_ranks: list[int], arena_numel: int, device):
        from torchtitan_b200.parallel.nvlink_comm import SymmetricHeap

        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.trainer_ranks, self.generator_ranks = trainer_ranks, generator_ranks
        self.heap = SymmetricHeap(group, 2 * arena_numel * 2 + (8 << 20), torch.device(device))
        self.half_off = [self.heap.alloc(arena_numel * 2, align=1024) for _ in range(2)]
        self.flag_off = [self.heap.alloc_flag() for _ in trainer_ranks]   # flag t: "trainer t finished version v"
        self.arena_numel = arena_numel
        self.version = 0
        self._segs = None
        self.bytes_pushed = 0

    def alloc(self, numel: int, dtype) -> torch.Tensor:
        """Allocator for ``ParamArena(alloc=...)`` on generator ranks: hands out the two heap halves in order."""
        assert numel == self.arena_numel and dtype == torch.bfloat16
        off = self.half_off[getattr(self, "_given", 0)]
        self._given = getattr(self, "_given", 0) + 1
        return self.heap.local_tensor(off, numel, dtype)

    # ---- trainer side ----------------------------------------------------------------------------------------------
    def build_plan(self, trainer_model: nn.Module, offsets: dict[str, int]) -> None:
        from torchtitan_b200.parallel import fsdp

        segs = []
        seen = set()
        units = fsdp.fsdp_units(trainer_model)
        name_of = {id(p): n for n, p in trainer_model.named_parameters()}
        for u in units:
            r = u.shard_rank
            for p in u.params:
                name = name_of.get(id(p.param), p.fqn)
                if name not in offsets or p.shard_dim != 0 or p.local_rows == 0:
                    if name in offsets and p.shard_dim != 0:
                        raise NotImplementedError(f"{name}: peer weight sync needs dim-0 shards")
                    continue
                src = u.shard_flat[p.shard_off : p.shard_off + p.local_rows * p.inner]
                assert src.dtype == torch.float32
                segs.append((src.data_ptr(), offsets[name] + r * p.chunk_rows * p.inner, p.local_rows * p.inner))
                seen.add(name)
        self._keep = units
        t = torch.tensor(segs, dtype=torch.int64)
        self._segs = t.to(self.heap.device)
        self.bytes_pushed = int(sum(s[2] for s in segs)) * 2 * len(self.generator_ranks)
        missing = [n for n in offsets if n not in seen]
        if missing and not units:
            raise NotImplementedError("peer weight sync needs FSDP units (fp32 master shards)")

    def push(self) -> None:
        """Trainer ranks: write version ``self.version + 1`` into the generators' inactive halves and publish it."""
        import ctypes

        from torchtitan_b200.ops import native
        from torchtitan_b200.parallel.nvlink_comm import _stream

        self.version += 1
        half = self.version % 2
        L = native.lib()
        ptrs = (ctypes.c_void_p * len(self.generator_ranks))(*[self.heap.peer_base[g] + self.half_off[half] for g in self.generator_ranks])
        native.check(L.tt_push_cast(self._segs.data_ptr(), self._segs.shape[0], ptrs, len(self.generator_ranks), _stream()), "tt_push_cast")
        me = self.trainer_ranks.index(self.rank)
        for g in self.generator_ranks:
            native.check(L.tt_set_flag(self.heap.peer_base[g] + self.flag_off[me], self.version, _stream()), "tt_set_flag")

    # ---- generator side -----------------------------------------------------------------------------------------------
    def wait_and_flip(self, arena: "ParamArena") -> None:
        import ctypes

        from torchtitan_b200.ops import native
        from torchtitan_b200.parallel.nvlink_comm import _stream

        self.version += 1
        flags = (ctypes.c_void_p * len(self.trainer_ranks))(*[self.heap.base + off for off in self.flag_off])
        native.check(native.lib().tt_wait_flags(flags, len(self.trainer_ranks), self.version, _stream()), "tt_wait_flags")
        target = self.version % 2
        if arena.active != target:
            arena.flip()
