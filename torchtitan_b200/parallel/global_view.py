"""Layout-independent views of parameters for checkpoints.

Tensor-parallel and expert-parallel shards are plain local tensors inside this framework (the FSDP runtime shards them
once more over the data-parallel ranks), so a parameter seen through ``module.state_dict()`` has the shape of its
tensor-parallel shard. A checkpoint must instead hold the FULL logical tensor, cut into per-rank pieces, so that it can be
loaded on any other layout and is interchangeable with checkpoints whose parameters are DTensors over the whole mesh
(torchtitan/components/checkpoint.py:60-100 saves the model's DTensor state dict as it is).

``global_view(param, tensor)`` wraps the local storage of ``tensor`` (the parameter itself or an optimizer state of the
same layout) in a DTensor over the combined mesh ``(outer shardings..., data-parallel mesh)`` with the full shape. Nothing
is copied: distributed-checkpoint loads write straight into the parameter's storage.

The order of the mesh dimensions is the order in which the tensor was cut: a column-parallel weight is split by tensor
parallel first and by FSDP second, both on dim 0, which DTensor expresses as ``[Shard(0), Shard(0)]`` on a mesh whose
first dimension is the tensor-parallel one.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import DTensor, Replicate, Shard

__all__ = ["global_view", "local_of", "is_outer_sharded"]

_MESHES: dict = {}


def is_outer_sharded(param) -> bool:
    return bool(getattr(param, "_tp_chain", None))


def _lines(mesh: DeviceMesh):
    """(size, stride, my coordinate) per dimension of ``mesh``; ranks along every dimension must be evenly spaced."""
    t, coord = mesh.mesh, mesh.get_coordinate()
    out = []
    for d in range(t.ndim):
        line = t[tuple(slice(None) if k == d else coord[k] for k in range(t.ndim))].tolist()
        stride = line[1] - line[0] if len(line) > 1 else 0
        if any(line[i] != line[0] + i * stride for i in range(len(line))):
            raise NotImplementedError(f"mesh dimension with unevenly spaced ranks {line}: cannot build a checkpoint view")
        out.append((len(line), stride, coord[d]))
    return out


def _combined_mesh(meshes: list[DeviceMesh]) -> DeviceMesh:
    key = tuple(id(m) for m in meshes)
    hit = _MESHES.get(key)
    if hit is not None:
        return hit[0]
    dims = [x for m in meshes for x in _lines(m)]
    base = dist.get_rank() - sum(c * s for _, s, c in dims)
    grid = torch.full([n for n, _, _ in dims], base, dtype=torch.int)
    for d, (n, s, _) in enumerate(dims):
        shape = [1] * len(dims)
        shape[d] = n
        grid = grid + (torch.arange(n, dtype=torch.int) * s).view(shape)
    names, seen = [], set()
    for m in meshes:
        for nm in (m.mesh_dim_names or tuple(f"dim{i}" for i in range(m.ndim))):
            while nm in seen:
                nm += "_"
            seen.add(nm)
            names.append(nm)
    groups = [g for m in meshes for g in m.get_all_groups()]
    mesh = DeviceMesh.from_group(groups, meshes[0].device_type, mesh=grid, mesh_dim_names=tuple(names))
    _MESHES[key] = (mesh, meshes)          # keep the source meshes alive: the key is made of their ids
    return mesh


def _contig_stride(shape):
    st, acc = [], 1
    for n in reversed(shape):
        st.append(acc)
        acc *= max(int(n), 1)
    return tuple(reversed(st))


def local_of(t):
    return t._local_tensor if isinstance(t, DTensor) else t


def global_view(param, tensor=None):
    """``tensor`` (default: ``param``) as a DTensor of the parameter's full logical shape, or unchanged when the parameter
    carries no tensor-/expert-parallel sharding."""
    tensor = param if tensor is None else tensor
    chain = getattr(param, "_tp_chain", None)
    if not chain:
        return tensor
    meshes = [m for _, m in chain]
    placements = [Shard(d) for d, _ in chain]
    if isinstance(param, DTensor):
        meshes.append(param.device_mesh)
        placements += list(param.placements)
    local = local_of(tensor)
    if local.dim() == 0 or tuple(local.shape) != tuple(local_of(param).shape):
        return tensor                                         # e.g. the scalar ``step`` of an optimizer state
    full = tuple(param._tp_full_shape)
    mesh = _combined_mesh(meshes)
    return DTensor.from_local(local.detach(), mesh, placements, run_check=False, shape=torch.Size(full),
                              stride=_contig_stride(full))
