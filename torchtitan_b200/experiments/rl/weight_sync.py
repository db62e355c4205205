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
    """The unsharded value of a (possibly FSDP- or tensor-parallel-sharded) parameter."""
    spec = getattr(p, "_tp_spec", None)
    t = p.full_tensor() if hasattr(p, "full_tensor") else p
    t = t.detach()
    if spec is not None and spec["placement"][0] == "shard":
        group, dim = spec["group"], spec["placement"][1]
        parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, t.contiguous(), group=group)
        t = torch.cat(parts, dim=dim)
    return t


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

    def __init__(self, model: nn.Module, double_buffer: bool = True):
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
        self.halves = [torch.zeros(off, dtype=p0.dtype, device=p0.device) for _ in range(2 if double_buffer else 1)]
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
