"""MoE data-movement and grouped-GEMM ops with autograd (CPU definitions; CUDA tensors take the
kernels in ``csrc/moe.cu`` through ``cuda_ops``)."""

from __future__ import annotations

import torch

from . import reference as ref


def route(x, gate_w, gate_b, expert_bias, **kw):
    if x.is_cuda:
        from . import cuda_ops

        return cuda_ops.moe_route(x, gate_w, gate_b, expert_bias, **kw)
    return ref.moe_route(x, gate_w, gate_b, expert_bias, **kw)


def sort_by_expert(expert_idx, num_experts: int):
    if expert_idx.is_cuda:
        from . import cuda_ops

        return cuda_ops.moe_sort(expert_idx, num_experts)
    return ref.moe_sort(expert_idx, num_experts)


def gather_rows(x, order, top_k: int):
    """rows[j] = x[order[j] // top_k]; backward scatter-adds (index_add) into x's gradient."""
    if x.is_cuda:
        from . import cuda_ops

        return cuda_ops.moe_gather_rows(x, order, top_k)
    return x[order // top_k]


def scale_rows(rows, scores_sorted, dispatcher=None, ctx=None):
    if ctx is not None and hasattr(dispatcher, "scale_rows"):
        return dispatcher.scale_rows(rows, scores_sorted, ctx)
    if rows.is_cuda:
        from . import cuda_ops

        return cuda_ops.scale_rows(rows, scores_sorted)
    return (rows.to(torch.float32) * scores_sorted.reshape(-1, 1)).to(rows.dtype)


def grouped_linear(x, w, counts):
    if x.is_cuda:
        from . import cuda_ops

        return cuda_ops.grouped_linear(x, w, counts)
    return _GroupedLinearRef.apply(x, w, counts)


class _GroupedLinearRef(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, counts):
        ctx.save_for_backward(x, w, counts)
        return ref.grouped_linear(x, w, counts)

    @staticmethod
    def backward(ctx, gy):
        x, w, counts = ctx.saved_tensors
        gx = torch.zeros_like(x)
        gw = torch.zeros_like(w)
        s = 0
        for e, n in enumerate(counts.tolist()):
            n = int(n)
            if n:
                g = gy[s : s + n]
                gx[s : s + n] = g @ w[e].to(g.dtype)
                gw[e] = (g.transpose(0, 1) @ x[s : s + n]).to(gw.dtype)
            s += n
        return gx, gw, None


def scatter_combine(rows, order, weights, num_tokens: int, top_k: int):
    """Undo the expert sort and reduce each token's k copies.

    ``rows`` [T*k, D] in sorted order; ``weights`` [T,k] fp32 or None (plain sum).
    out[t] = sum_s w[t,s] * rows[inv(t*k+s)], accumulated in fp32 when weighted.
    """
    if rows.is_cuda:
        from . import cuda_ops

        return cuda_ops.moe_scatter_combine(rows, order, weights, num_tokens, top_k)
    D = rows.shape[-1]
    unsorted = rows.new_zeros(num_tokens * top_k, D)
    unsorted[order] = rows[: order.numel()]
    unsorted = unsorted.view(num_tokens, top_k, D)
    if weights is None:
        return unsorted.sum(dim=1)
    return torch.bmm(weights.reshape(-1, 1, top_k), unsorted.float()).to(rows.dtype).squeeze(1)


class _AuxLoss(torch.autograd.Function):
    """Identity on x whose backward adds d(aux)/dx. aux = coeff * E * sum_e f_e * P_e with
    f_e the routed fraction (constant) and P_e the mean softmax probability of expert e."""

    @staticmethod
    def forward(ctx, x, gate_w, counts, coeff, top_k):
        ctx.save_for_backward(x, gate_w, counts)
        ctx.coeff, ctx.top_k = coeff, top_k
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        x, gate_w, counts = ctx.saved_tensors
        T, E = x.shape[0], gate_w.shape[0]
        with torch.enable_grad():
            xd = x.detach().float().requires_grad_(True)
            wd = gate_w.detach().float().requires_grad_(True)
            p = torch.softmax(xd @ wd.t(), dim=-1).mean(0)
            f = counts.float() / (T * ctx.top_k)
            aux = ctx.coeff * E * (f * p).sum()
            gx, gw = torch.autograd.grad(aux, (xd, wd))
        return g + gx.to(g.dtype), gw.to(gate_w.dtype), None, None, None


def inject_aux_loss(x, gate_w, counts, coeff: float, top_k: int):
    return _AuxLoss.apply(x, gate_w, counts, coeff, top_k)
