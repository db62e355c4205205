"""``ParallelDims``: validates the parallel degrees and answers "which ranks share dimension X
with me" for the three views of the world that a job needs.

Same three factorizations of ``range(world_size)`` as torchtitan/distributed/parallel_dims.py:68-189
(row-major, left-most slowest):

* data loading ``[pp, batch, cp, tp]``            with ``batch = dp_replicate * dp_shard``
* dense params ``[pp, dp_replicate, fsdp, tp]``   with ``fsdp  = dp_shard * cp``
* sparse params ``[pp, dp_replicate, efsdp, ep, etp]`` with ``efsdp = fsdp * tp / (ep * etp)``
* ``loss`` = ``batch`` and ``cp`` flattened (every rank that sees different data).

The rank arithmetic (:class:`RankGrid`) is pure Python, so layouts can be checked for any
world size without creating process groups. Groups are created lazily, once per distinct
rank set (two dimensions with identical rank sets share one group), and wrapped into a
``DeviceMesh`` because DTensor/DCP need that type. Dimensions of size 1 never get a group.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from torchtitan_b200.tools.logging import logger
from torchtitan_b200.tools.utils import device_type

__all__ = ["ParallelDims", "RankGrid"]


class RankGrid:
    """A row-major factorization of ``range(world)`` into named dimensions."""

    def __init__(self, names: tuple[str, ...], sizes: tuple[int, ...]):
        assert len(names) == len(sizes)
        self.names, self.sizes = tuple(names), tuple(int(s) for s in sizes)
        self.world = math.prod(self.sizes)
        self.strides = tuple(
            math.prod(self.sizes[i + 1 :]) for i in range(len(self.sizes))
        )

    def coords(self, rank: int) -> dict[str, int]:
        return {
            n: (rank // st) % sz for n, st, sz in zip(self.names, self.strides, self.sizes)
        }

    def group_ranks(self, rank: int, dims: tuple[str, ...]) -> list[int]:
        """Ranks that differ from ``rank`` only along ``dims`` (ordered with ``dims`` as a
        row-major sub-grid in the order the grid declares them)."""
        idx = [self.names.index(d) for d in dims]
        idx.sort()
        base = rank
        for i in idx:
            base -= ((rank // self.strides[i]) % self.sizes[i]) * self.strides[i]
        out = [base]
        for i in idx:
            out = [r + k * self.strides[i] for r in out for k in range(self.sizes[i])]
        return out

    def all_groups(self, dims: tuple[str, ...]) -> list[list[int]]:
        seen, groups = set(), []
        for r in range(self.world):
            g = self.group_ranks(r, dims)
            if g[0] not in seen and tuple(g) not in seen:
                seen.add(tuple(g))
                seen.add(g[0]) if False else None
                groups.append(g)
        # dedupe while keeping first-rank order
        uniq, keys = [], set()
        for g in groups:
            k = tuple(g)
            if k not in keys:
                keys.add(k)
                uniq.append(g)
        return uniq


_MESH_NAMES = (
    "pp", "batch", "loss", "dp_replicate", "fsdp", "cp", "tp", "ep", "efsdp", "etp",
)


@dataclass
class ParallelDims:
    dp_replicate: int
    dp_shard: int
    cp: int
    tp: int
    pp: int
    ep: int
    etp: int
    world_size: int

    _meshes: dict = field(default_factory=dict, repr=False)
    _groups: dict = field(default_factory=dict, repr=False)
    _world_mesh: object = field(default=None, repr=False)

    def __post_init__(self):
        self._validate()

    # ------------------------------------------------------------------ validation
    def _validate(self):
        for d in (self.dp_replicate, self.cp, self.tp, self.pp, self.ep, self.etp):
            assert d >= 1, "Parallelism degree should be >= 1, except for dp_shard"
        assert self.dp_shard == -1 or self.dp_shard >= 1, "dp_shard must -1 or >=1."
        rest = self.dp_replicate * self.cp * self.tp * self.pp
        if self.dp_shard < 0:
            self.dp_shard = self.world_size // rest
        assert self.dp_shard >= 1
        assert rest * self.dp_shard == self.world_size, (
            f"Invalid parallel dims: dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * "
            f"cp({self.cp}) * tp({self.tp}) * pp({self.pp}) != WORLD_SIZE({self.world_size})"
        )
        if self.ep > 1:
            assert self.etp == self.tp or self.etp == 1, "Currently we only support ETP=TP or ETP=1"
            assert (self.dp_shard * self.cp * self.tp) % (self.ep * self.etp) == 0, (
                f"ep({self.ep}) * etp({self.etp}) must divide dp_shard*cp*tp"
            )

    # ------------------------------------------------------------------ rank grids
    @property
    def grids(self) -> dict[str, RankGrid]:
        batch = self.dp_replicate * self.dp_shard
        fsdp = self.dp_shard * self.cp
        ep_span = self.ep * self.etp
        efsdp = max(1, fsdp * self.tp // ep_span)
        return {
            "dataloading": RankGrid(("pp", "batch", "cp", "tp"), (self.pp, batch, self.cp, self.tp)),
            "dense": RankGrid(("pp", "dp_replicate", "fsdp", "tp"), (self.pp, self.dp_replicate, fsdp, self.tp)),
            "sparse": RankGrid(
                ("pp", "dp_replicate", "efsdp", "ep", "etp"),
                (self.pp, self.dp_replicate, efsdp, self.ep, self.etp),
            ),
        }

    def _dim_home(self, name: str) -> tuple[str, tuple[str, ...]]:
        home = {
            "pp": ("dataloading", ("pp",)),
            "batch": ("dataloading", ("batch",)),
            "cp": ("dataloading", ("cp",)),
            "tp": ("dataloading", ("tp",)),
            "loss": ("dataloading", ("batch", "cp")),
            "dp_replicate": ("dense", ("dp_replicate",)),
            "fsdp": ("dense", ("fsdp",)),
            "ep": ("sparse", ("ep",)),
            "efsdp": ("sparse", ("efsdp",)),
            "etp": ("sparse", ("etp",)),
        }
        if name not in home:
            raise ValueError(f"Invalid mesh dim: '{name}'. Valid dimensions are: {list(_MESH_NAMES)}")
        return home[name]

    def dim_size(self, name: str) -> int:
        grid, dims = self._dim_home(name)
        g = self.grids[grid]
        return math.prod(g.sizes[g.names.index(d)] for d in dims)

    def ranks_of(self, name: str, rank: int) -> list[int]:
        """Ranks in ``rank``'s group along mesh dimension ``name`` (no process group needed)."""
        grid, dims = self._dim_home(name)
        return self.grids[grid].group_ranks(rank, dims)

    def coordinate(self, name: str, rank: int) -> int:
        return self.ranks_of(name, rank).index(rank)

    def _mesh_exist(self, name: str, degree: int) -> bool:
        if name == "efsdp":
            return self.ep > 1
        return degree > 1

    # ------------------------------------------------------------------ process groups
    def _device_type(self) -> str:
        return device_type

    # A job may give the dims only a subset of its ranks (e.g. the trainer ranks of an RL job whose other ranks generate):
    # ``set_base_ranks`` maps grid positions 0..world_size-1 to those global ranks. Process-group creation stays a
    # collective of the whole job, so the ranks outside the subset must call ``build_mesh()`` on an identical object
    # (they become members of no group).
    def set_base_ranks(self, ranks: list[int] | None) -> None:
        assert ranks is None or len(ranks) == self.world_size
        self._base = list(ranks) if ranks is not None else None
        self._meshes, self._groups = {}, {}

    def _global(self, ranks: list[int]) -> list[int]:
        base = getattr(self, "_base", None)
        return list(ranks) if base is None else [base[r] for r in ranks]

    def _me(self) -> int:
        """This process's position in the grids."""
        base = getattr(self, "_base", None)
        return dist.get_rank() if base is None else base.index(dist.get_rank())

    def _new_group(self, granks: list[int]):
        if getattr(self, "_base", None) is None:
            return dist.new_group(granks)
        key = ("sub",) + tuple(granks)            # one group per distinct rank set
        if key not in self._groups:
            self._groups[key] = dist.new_group(granks)
        return self._groups[key]

    def _group_for(self, grid_name: str, dims: tuple[str, ...]):
        """Create (collectively, on every rank) the groups of one dimension; return mine."""
        grid = self.grids[grid_name]
        mine = None
        me = dist.get_rank()
        whole_job = getattr(self, "_base", None) is None
        for ranks in grid.all_groups(dims):
            granks = self._global(ranks)
            key = tuple(granks)
            if key not in self._groups:
                if whole_job and len(ranks) == self.world_size and ranks == list(range(self.world_size)):
                    self._groups[key] = dist.group.WORLD
                else:
                    self._groups[key] = self._new_group(granks)
            if me in granks:
                mine = (self._groups[key], granks)
        assert mine is not None or getattr(self, "_base", None) is not None
        return mine

    def build_mesh(self):
        """Create every enabled dimension's group and ``DeviceMesh`` (collective call)."""
        from torch.distributed.device_mesh import DeviceMesh

        logger.info(
            f"Building device mesh with parallelism: pp={self.pp}, dp_replicate={self.dp_replicate}, "
            f"dp_shard={self.dp_shard}, cp={self.cp}, tp={self.tp}, ep={self.ep}, etp={self.etp}"
        )
        assert dist.is_initialized(), "init_distributed() must run before build_mesh()"
        base = getattr(self, "_base", None)
        assert base is not None or dist.get_world_size() == self.world_size, (
            f"world size {dist.get_world_size()} != ParallelDims.world_size {self.world_size}"
        )
        dev = self._device_type()
        self._meshes = {}
        for name in _MESH_NAMES:
            size = self.dim_size(name)
            if not self._mesh_exist(name, size):
                self._meshes[name] = None
                continue
            grid_name, dims = self._dim_home(name)
            if size == 1:  # efsdp of size 1 under EP: a one-rank group
                pg, ranks = None, [dist.get_rank()]
                # every rank must take part in new_group calls: make them all
                for r in self._global(list(range(self.world_size))):
                    g = self._new_group([r])
                    if r == dist.get_rank():
                        pg = g
            else:
                got = self._group_for(grid_name, dims)
                if got is None:              # this rank is outside the subset: it only took part in the creation
                    self._meshes[name] = None
                    continue
                pg, ranks = got
            if base is not None and dist.get_rank() not in base:
                self._meshes[name] = None
                continue
            self._meshes[name] = DeviceMesh.from_group(
                pg, dev, mesh=torch.tensor(ranks, dtype=torch.int), mesh_dim_names=(name,)
            )
        all_ranks = self._global(list(range(self.world_size)))
        world_pg = dist.group.WORLD if base is None else self._new_group(all_ranks)
        if base is not None and dist.get_rank() not in base:
            self._world_mesh = None
            return None
        self._world_mesh = DeviceMesh.from_group(
            world_pg, dev, mesh=torch.tensor(all_ranks, dtype=torch.int), mesh_dim_names=("world",)
        )
        active = [k for k, v in self._meshes.items() if v is not None]
        logger.info(f"Successfully created meshes with active dimensions: {active}")
        return self._world_mesh

    # ------------------------------------------------------------------ mesh access
    def get_optional_mesh(self, dims: str | list[str]):
        if isinstance(dims, str):
            dims = [dims]
        for d in dims:
            if d not in _MESH_NAMES:
                raise ValueError(f"Invalid mesh dim: '{d}'. Valid dimensions are: {list(_MESH_NAMES)}")
        if any(not self._mesh_exist(d, self.dim_size(d)) for d in dims):
            return None
        if not self._meshes:
            self.build_mesh()
        if len(dims) == 1:
            return self._meshes[dims[0]]
        return self._multi_dim_mesh(tuple(dims))

    def _multi_dim_mesh(self, dims: tuple[str, ...]):
        from torch.distributed.device_mesh import DeviceMesh

        key = ("nd",) + dims
        if key in self._meshes:
            return self._meshes[key]
        homes = {self._dim_home(d)[0] for d in dims}
        for grid_name, grid in self.grids.items():
            if all(d in grid.names for d in dims):
                break
        else:
            raise ValueError(f"Invalid mesh name combinations {list(dims)} (homes {homes}).")
        ranks = self._global(grid.group_ranks(self._me(), dims))
        order = sorted(dims, key=grid.names.index)
        if list(order) != list(dims):
            raise ValueError(f"mesh dims must be requested in grid order {order}, got {list(dims)}")
        shape = [grid.sizes[grid.names.index(d)] for d in dims]
        pgs = [self._meshes[d].get_group() for d in dims]
        mesh = DeviceMesh.from_group(
            pgs, self._device_type(), mesh=torch.tensor(ranks, dtype=torch.int).view(shape), mesh_dim_names=dims
        )
        self._meshes[key] = mesh
        return mesh

    def get_mesh(self, dims: str | list[str]):
        mesh = self.get_optional_mesh(dims)
        if mesh is None:
            how = "enabled (size > 1)" if isinstance(dims, str) else "all enabled"
            raise ValueError(
                f"Mesh '{dims}' is not available. Ensure the corresponding parallelism dimension is {how}."
            )
        return mesh

    def get_all_one_dimensional_meshes(self) -> dict:
        if not self._meshes:
            self.build_mesh()
        return {
            k: v for k, v in self._meshes.items()
            if isinstance(k, str) and v is not None and v.ndim == 1 and v.size() > 1
        }

    @property
    def world_mesh(self):
        if self._world_mesh is None:
            self.build_mesh()
        return self._world_mesh

    # ------------------------------------------------------------------ flags
    @property
    def dp_enabled(self): return self.dp_replicate > 1 or self.dp_shard > 1
    @property
    def dp_replicate_enabled(self): return self.dp_replicate > 1
    @property
    def dp_shard_enabled(self): return self.dp_shard > 1
    @property
    def cp_enabled(self): return self.cp > 1
    @property
    def dp_cp_enabled(self): return self.dp_enabled or self.cp_enabled
    @property
    def fsdp_enabled(self): return self.dp_shard_enabled or self.cp_enabled
    @property
    def tp_enabled(self): return self.tp > 1
    @property
    def pp_enabled(self): return self.pp > 1
    @property
    def ep_enabled(self): return self.ep > 1
    @property
    def etp_enabled(self): return self.etp > 1

    @property
    def fsdp_gradient_divide_factor(self) -> int:
        """All ranks that see different data: the divisor FSDP would apply if the loss were not
        already normalised by the global token count."""
        return self.dp_replicate * self.dp_shard * self.cp

    @property
    def non_data_parallel_size(self) -> int:
        return self.cp * self.tp * self.pp

    @property
    def seq_len_divisor(self) -> int:
        """Sequence parallel shards by tp; head-tail context parallel needs 2*cp chunks."""
        return self.tp * (self.cp * 2)
