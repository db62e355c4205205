"""Expert parallelism for MoE layers.

Reference behaviour (torchtitan/distributed/expert_parallel.py:28-285 and the wiring in
torchtitan/models/llama4/parallelize.py:525-630): expert weights are sharded on the expert dimension
over the ``ep`` mesh; *dispatch* exchanges per-expert token counts, then the token rows, with
all-to-all collectives and regroups the received rows by local expert (padded to the grouped-GEMM
alignment); *combine* undoes both. With tensor parallel and ``etp = 1`` each TP rank routes only its
own sequence shard (the "reorderer sequence parallel" arrangement), so nothing is gathered around
the MoE layer; the router and (without EP) the expert weights are then replicated over TP and their
gradients are summed over the TP group.

Here the MoE layer itself contains no distributed code: ``GroupedExperts.dispatcher`` is swapped
for :class:`AllToAllDispatcher`. Under FSDP the routed experts form their own unit on the ``efsdp``
mesh (``efsdp = fsdp * tp / (ep * etp)``), the rest of the block is sharded over ``fsdp``
(MoE-aware FSDP, torchtitan/models/llama4/parallelize.py:349-522).
``expert_parallel_comm_backend = deepep | hybridep`` selects the same dispatcher with the
capacity-factor (sync-free, fixed-size buffers) mode when
``hybridep_non_blocking_expert_capacity_factor`` is set.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from torchtitan_b200.models.common.moe.permute import generate_permute_indices
from torchtitan_b200.tools.logging import logger

__all__ = ["apply_moe_ep_tp", "AllToAllDispatcher", "all_to_all_rows"]


def _exchange(out, x, out_splits, in_splits, group):
    """The all-to-all itself. Inside a pipeline slot that runs a forward and a backward together
    (``parallel/overlap.py``) it is issued in the background and the other piece of work gets the compute stream until
    its own next exchange; the wait comes after the baton is back."""
    from . import overlap

    if overlap.active():
        work = dist.all_to_all_single(out, x, out_splits, in_splits, group=group, async_op=True)
        overlap.yield_point()
        work.wait()
    else:
        dist.all_to_all_single(out, x, out_splits, in_splits, group=group)
    return out


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all of rows; backward runs the reverse exchange."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        return _exchange(out, x.contiguous(), out_splits, in_splits, group)

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        return _exchange(out, g.contiguous(), ctx.in_splits, ctx.out_splits, ctx.group), None, None, None


def all_to_all_rows(x, out_splits, in_splits, group):
    return _AllToAllRows.apply(x, list(out_splits), list(in_splits), group)


class AllToAllDispatcher:
    """Token exchange for expert parallel (``standard`` backend).

    ``alignment``: every local expert's block of rows is padded to a multiple of it (8 for bf16, 16
    for float8, 32 for MXFP8 grouped GEMMs). ``capacity_factor``: when set, receive buffers have the
    fixed size ``tokens * top_k * factor`` rows per source rank and rows beyond it are dropped, which
    removes the device-to-host read of the split sizes."""

    def __init__(self, ep_mesh, num_experts: int, alignment: int = 8, capacity_factor: float | None = None):
        self.group = ep_mesh.get_group()
        self.ep, self.rank = ep_mesh.size(), ep_mesh.get_local_rank()
        assert num_experts % self.ep == 0, f"ep ({self.ep}) must divide num_experts ({num_experts})"
        self.num_experts, self.local_experts = num_experts, num_experts // self.ep
        self.alignment, self.capacity_factor = alignment, capacity_factor

    def dispatch(self, x, order, counts, top_k: int):
        if x.is_cuda:
            from torchtitan_b200.ops.cuda_ops import moe_gather_rows

            rows = moe_gather_rows(x, order, top_k)   # sorted by global expert => contiguous per destination rank
        else:
            rows = x[order // top_k]
        counts = counts.to(torch.int64)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.group)  # [src rank][local expert]
        in_splits = counts.view(self.ep, self.local_experts).sum(1).tolist()
        out_splits = recv_counts.view(self.ep, self.local_experts).sum(1).tolist()
        recv = all_to_all_rows(rows, out_splits, in_splits, self.group)
        n_recv = recv.shape[0]
        max_len = n_recv + self.local_experts * self.alignment
        max_len = -(-max_len // self.alignment) * self.alignment      # the quantised grouped GEMM wants whole row blocks
        perm, m_sizes, _ = generate_permute_indices(
            recv_counts.to(torch.int32), self.local_experts, self.ep, max_len, self.alignment, use_cpu=not recv.is_cuda)
        perm = perm.to(recv.device).long()
        padded = torch.vstack((recv, recv.new_zeros(1, recv.shape[-1])))  # index -1 -> the zero row
        grouped = padded[perm]
        ctx = {"perm": perm, "n_recv": n_recv, "in_splits": in_splits, "out_splits": out_splits, "rows": rows.shape[0]}
        sizes = m_sizes.to(torch.int64).to(recv.device)
        sizes._tt_aligned = self.alignment      # read by the CUDA grouped GEMM wrapper (needs multiples of 64)
        return grouped, sizes, ctx

    def scale_rows(self, rows, scores_sorted, ctx):
        # scores travel with the rows: exchange and permute them the same way
        sc = all_to_all_rows(scores_sorted.reshape(-1, 1).float(), ctx["out_splits"], ctx["in_splits"], self.group)
        sc = torch.vstack((sc, sc.new_zeros(1, 1)))[ctx["perm"]]
        if rows.is_cuda:
            from torchtitan_b200.ops.cuda_ops import scale_rows

            return scale_rows(rows, sc)
        return (rows.float() * sc).to(rows.dtype)

    def combine(self, y, ctx):
        perm = ctx["perm"]
        out = y.new_zeros(ctx["n_recv"] + 1, y.shape[-1])
        out = out.index_copy(0, torch.where(perm >= 0, perm, torch.full_like(perm, ctx["n_recv"])), y)
        out = out[: ctx["n_recv"]]
        return all_to_all_rows(out, ctx["in_splits"], ctx["out_splits"], self.group)


def _shard_experts(experts: nn.Module, ep_mesh) -> None:
    W, r, group = ep_mesh.size(), ep_mesh.get_local_rank(), ep_mesh.get_group()
    for name in ("w1", "w2", "w3", "b1", "b2", "b3", "mlp1_weight", "mlp1_bias", "mlp2_weight", "mlp2_bias"):
        p = experts._parameters.get(name)
        if p is None:
            continue
        E = p.shape[0]
        n = E // W
        if p.device.type == "meta":
            local = torch.empty((n,) + tuple(p.shape[1:]), dtype=p.dtype, device="meta")
        else:
            local = p.detach()[r * n : (r + 1) * n].clone()
        newp = nn.Parameter(local, requires_grad=p.requires_grad)
        spec = {"placement": ("shard", 0), "group": group, "mesh": ep_mesh, "full_shape": tuple(p.shape)}
        experts.__dict__.setdefault("_tp_specs", {})[name] = spec  # same tagging protocol as tensor parallel
        from .tp import _tag

        _tag(newp, spec)
        experts._parameters[name] = newp
    experts.num_local_experts = experts.w1.shape[0] if hasattr(experts, "w1") else None


class _GatherRows(torch.autograd.Function):
    """Concatenate the ranks' row blocks [T, D] -> [W * T, D]; backward sums the ranks' gradients of each block."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = dist.get_world_size(group)
        x = x.contiguous()
        out = x.new_empty((W * x.shape[0],) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        W = dist.get_world_size(ctx.group)
        g = g.contiguous()
        out = g.new_empty((g.shape[0] // W,) + tuple(g.shape[1:]))
        dist.reduce_scatter_tensor(out, g, group=ctx.group)
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    """Sum the ranks' [W * T, D] partial results and keep this rank's block [T, D]; backward gathers."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = dist.get_world_size(group)
        x = x.contiguous()
        out = x.new_empty((x.shape[0] // W,) + tuple(x.shape[1:]))
        dist.reduce_scatter_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        W = dist.get_world_size(ctx.group)
        g = g.contiguous()
        out = g.new_empty((W * g.shape[0],) + tuple(g.shape[1:]))
        dist.all_gather_into_tensor(out, g, group=ctx.group)
        return out, None


def gather_rows(x, group):
    return _GatherRows.apply(x, group)


def reduce_scatter_rows(x, group):
    return _ReduceScatterRows.apply(x, group)


def _shard_experts_hidden(experts: nn.Module, etp_mesh) -> None:
    """Expert tensor parallel: split every expert's hidden dimension over ``etp_mesh`` (``w1``/``w3`` [E, H, D] by rows,
    ``w2`` [E, D, H] by columns), so a rank produces partial sums of the expert outputs.
    Parity: ExpertTensorParallel, torchtitan/distributed/expert_parallel.py (2-D expert sharding [ep, etp])."""
    W, r, group = etp_mesh.size(), etp_mesh.get_local_rank(), etp_mesh.get_group()
    if not all(hasattr(experts, n) for n in ("w1", "w2", "w3")) or any(
            experts._parameters.get(n) is not None for n in ("mlp1_weight", "mlp1_bias", "b1")):
        raise NotImplementedError("expert tensor parallel covers SwiGLU experts without biases (w1 / w2 / w3)")
    for name, dim in (("w1", 1), ("w3", 1), ("w2", 2)):
        p = experts._parameters[name]
        assert p.shape[dim] % W == 0, f"{name}: hidden size {p.shape[dim]} not divisible by etp={W}"
        n = p.shape[dim] // W
        if p.device.type == "meta":
            shape = list(p.shape)
            shape[dim] = n
            local = torch.empty(shape, dtype=p.dtype, device="meta")
        else:
            local = p.detach().narrow(dim, r * n, n).clone()
        newp = nn.Parameter(local, requires_grad=p.requires_grad)
        prev = experts.__dict__.get("_tp_specs", {}).get(name)
        groups = ((prev["group"],) if prev is not None else ()) + (group,)
        spec = {"placement": ("shard", dim), "group": group, "mesh": etp_mesh,
                "full_shape": tuple(prev["full_shape"] if prev is not None else p.shape), "norm_groups": groups,
                "outer": prev}
        experts.__dict__.setdefault("_tp_specs", {})[name] = spec
        from .tp import _tag

        _tag(newp, spec)
        newp._extra_norm_groups = groups       # the squared norm is a partial sum over both the ep and the etp group
        experts._parameters[name] = newp


def apply_moe_ep_tp(model: nn.Module, parallel_dims, parallelism) -> nn.Module:
    from .tp import _mark_replicated

    ep_mesh = parallel_dims.get_optional_mesh("ep")
    tp_mesh = parallel_dims.get_optional_mesh("tp")
    etp_mesh = parallel_dims.get_optional_mesh("etp") if parallel_dims.etp_enabled else None
    if parallel_dims.etp_enabled and tp_mesh is None:
        raise ValueError("expert tensor parallel needs tensor parallel (etp must equal tp)")
    from torchtitan_b200.models.common.moe.moe import GROUP_ALIGN_NATIVE, group_alignment
    from torchtitan_b200.ops import native

    # 64-row groups let the device-side grouped GEMM (incl. its weight-gradient form) run without host-side sizes
    alignment = GROUP_ALIGN_NATIVE if (torch.cuda.is_available() and native.has("tt_grouped_gemm")) else 8
    cf = parallelism.hybridep_non_blocking_expert_capacity_factor if parallelism is not None else None
    # 'deepep' / 'hybridep' select the peer-memory dispatch / combine kernels (no external library); they need every rank
    # of the expert-parallel group on one NVLink domain, else the collective dispatcher is used
    nvlink_ep = False
    if ep_mesh is not None and getattr(parallelism, "expert_parallel_comm_backend", "standard") in ("deepep", "hybridep"):
        from .nvlink_ep import NvlinkDispatcher

        nvlink_ep = NvlinkDispatcher.available(ep_mesh)
        if not nvlink_ep:
            logger.info("expert_parallel_comm_backend: peer-memory dispatch unavailable here; using all-to-all collectives")
    n = 0
    for block in model.layers.values():
        if not getattr(block, "moe_enabled", False):
            continue
        moe = block.moe
        n += 1
        if tp_mesh is not None:
            # sequence-sharded tokens are routed by their own TP rank; everything in the MoE layer that is not
            # expert-sharded is replicated over TP and accumulates partial gradients
            for sub in (moe.router.gate, moe.shared_experts):
                if sub is not None:
                    for m in sub.modules():
                        _mark_replicated(m, tp_mesh.get_group(), tp_mesh)
            if ep_mesh is None:
                _mark_replicated(moe.experts, tp_mesh.get_group(), tp_mesh)
        if ep_mesh is not None:
            _shard_experts(moe.experts, ep_mesh)
            if nvlink_ep:
                from .nvlink_ep import NvlinkDispatcher

                moe.experts.dispatcher = NvlinkDispatcher(ep_mesh, moe.router.num_experts,
                                                          alignment=group_alignment(moe.experts, GROUP_ALIGN_NATIVE),
                                                          capacity_factor=cf)
            else:
                moe.experts.dispatcher = AllToAllDispatcher(ep_mesh, moe.router.num_experts,
                                                            alignment=group_alignment(moe.experts, alignment),
                                                            capacity_factor=cf)
        if etp_mesh is not None:
            if moe.aux_loss_coeff > 0.0:
                raise NotImplementedError("the auxiliary load-balance loss is not supported with expert tensor parallel")
            _shard_experts_hidden(moe.experts, etp_mesh)
            moe._etp_group = etp_mesh.get_group()
    if n:
        logger.info(f"Applied expert parallel to {n} MoE layers (ep={parallel_dims.ep}, backend={getattr(parallelism, 'expert_parallel_comm_backend', 'standard')})")
    return model
