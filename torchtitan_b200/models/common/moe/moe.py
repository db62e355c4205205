"""Mixture-of-experts layer: router -> dispatch -> grouped SwiGLU experts -> combine.

Semantics follow torchtitan/models/common/moe/moe.py:24-579:

* ``GroupedExperts``: 3-D parameters ``w1[E,H,D] w2[E,D,H] w3[E,H,D]`` (names kept for
  checkpoints), output ``(silu(x w1^T) * x w3^T) w2^T`` per expert group (:24-127).
* ``TokenChoiceTopKRouter``: gate in fp32, softmax or sigmoid scores, ``expert_bias`` added
  only for *choosing* experts, optional node-limited routing (keep ``num_limited_groups``
  groups ranked by the sum of their top-2 scores), ``route_norm`` and ``route_scale``, a
  round-robin debug mode, and a per-expert token histogram (:130-326).
* ``MoE``: shared experts as one wide FeedForward, ``score_before_experts`` (scale the routed
  rows) or after (weighted sum over the k copies in fp32), persistent ``expert_bias`` and
  non-persistent ``tokens_per_expert`` buffers (:373-579).

Structure differs: the (token, slot) pairs are placed by a counting sort (``ops.moe_sort``)
and all movement of rows goes through a *dispatcher* object owned by ``GroupedExperts``
(``LocalDispatcher`` here; expert parallel installs its own in ``parallel/ep.py``), so the
layer body has no distributed code and no host synchronisation.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

import torch
import torch.nn as nn

from torchtitan_b200 import ops
from torchtitan_b200.ops import reference as ref
from torchtitan_b200.protocols.module import Module

from ..feed_forward import FeedForward
from ..linear import Linear


def _moe_ops():
    from torchtitan_b200.ops import moe_ops

    return moe_ops


GROUP_ALIGN_NATIVE = 64  # contraction tile of the grouped weight-gradient kernel
GROUP_ALIGN_MX_NATIVE = 128  # row block of the block-scaled grouped GEMM's scale layout (and its contraction tile)


def group_alignment(experts, base: int) -> int:
    """Rows every expert's block is padded to: ``base`` from the dispatcher's own needs, raised to what the experts'
    quantised grouped GEMM wants (MXFP8 on the native kernel: 128; otherwise the recipe's block along the tokens)."""
    from . import utils as _utils

    base = max(base, _utils.TOKEN_GROUP_ALIGN_SIZE_M)      # floor set through set_token_group_alignment_size_m
    quant = getattr(experts, "quant", None)
    if quant is None:
        return base
    if quant.kind == "mxfp8":
        from torchtitan_b200.ops import native

        need = GROUP_ALIGN_MX_NATIVE if (torch.cuda.is_available() and not quant.emulate and native.has("tt_grouped_gemm_mxfp8")) else 32
    else:
        need = 16
    return max(base, need) if max(base, need) % min(base, need) == 0 else base * need


class LocalDispatcher:
    """All experts live on this rank: dispatch = gather rows in expert order.

    With ``alignment > 1`` every expert's block of rows starts at a multiple of ``alignment`` (zero rows in between),
    which is what the device-side grouped GEMM needs; the layout is computed on the device from the counts, so there is
    no host synchronisation. ``alignment=None`` picks 64 for CUDA bf16 inputs when the native kernel is built, else 1."""

    def __init__(self, alignment: int | None = None):
        self.alignment = alignment

    def _align_for(self, x) -> int:
        if self.alignment is not None:
            return self.alignment
        if x.is_cuda and x.dtype == torch.bfloat16:
            from torchtitan_b200.ops import native

            return GROUP_ALIGN_NATIVE if native.has("tt_grouped_gemm") else 1
        return 1

    def dispatch(self, x, order, counts, top_k: int):
        a = self._align_for(x)
        if a <= 1:
            return _moe_ops().gather_rows(x, order, top_k), counts, None
        n, E = order.numel(), counts.numel()
        c = counts.to(torch.int64)
        padded = (c + (a - 1)) // a * a
        starts = torch.cumsum(c, 0) - c
        pstarts = torch.cumsum(padded, 0) - padded
        jpos = torch.arange(n, device=x.device)
        expert = torch.searchsorted(torch.cumsum(c, 0), jpos, right=True).clamp_(max=E - 1)
        dest = jpos + (pstarts - starts)[expert]                # padded row of sorted entry j
        max_rows = (n + E * (a - 1) + a - 1) // a * a          # static upper bound on the padded row count
        pc = padded.to(counts.dtype)
        pc._tt_aligned = a                                      # read by the CUDA grouped GEMM wrapper
        ctx = {"dest": dest, "max_rows": max_rows}
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
            # one gather straight into the padded layout; `pair` / `pos` are the row <-> (token, slot) maps
            pair = torch.full((max_rows,), -1, dtype=torch.int64, device=x.device).index_copy_(0, dest, order)
            pos = torch.empty(n, dtype=torch.int32, device=x.device).index_copy_(0, order, dest.to(torch.int32))
            src = torch.where(pair >= 0, pair // top_k, pair).to(torch.int32)
            ctx.update(pair=pair, pos=pos, top_k=top_k, tokens=x.shape[0])
            from torchtitan_b200.ops import cuda_ops

            return cuda_ops.moe_gather_src(x, src, pos, top_k), pc, ctx
        rows = x.new_zeros(max_rows, x.shape[-1]).index_copy(0, dest, _moe_ops().gather_rows(x, order, top_k))
        return rows, pc, ctx

    def scale_rows(self, rows, scores_sorted, ctx):
        sc = rows.new_zeros(ctx["max_rows"], 1, dtype=torch.float32).index_copy(0, ctx["dest"], scores_sorted.reshape(-1, 1).float())
        if rows.is_cuda:
            from torchtitan_b200.ops.cuda_ops import scale_rows

            return scale_rows(rows, sc)
        return (rows.float() * sc).to(rows.dtype)

    def combine(self, y, ctx):
        return y if ctx is None else y.index_select(0, ctx["dest"])

    def combine_to_tokens(self, y, weights, ctx):
        """Fused un-pad + un-sort + weighted sum over the k copies (CUDA bf16 path); None when not applicable."""
        if ctx is None or "pos" not in ctx or y.dtype != torch.bfloat16:
            return None
        from torchtitan_b200.ops import cuda_ops

        return cuda_ops.moe_combine_pos(y, ctx["pos"], ctx["pair"], weights, ctx["tokens"], ctx["top_k"])


class GroupedExperts(Module):
    def __init__(self, *, dim: int, hidden_dim: int, num_experts: int, use_grouped_mm: bool):
        super().__init__()
        self.num_experts = num_experts
        self.w1 = nn.Parameter(torch.empty(num_experts, hidden_dim, dim))
        self.w2 = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.w3 = nn.Parameter(torch.empty(num_experts, hidden_dim, dim))
        self.use_grouped_mm = use_grouped_mm
        self.dispatcher = LocalDispatcher()
        self.quant = None  # a QuantRecipe once a quantisation converter selected these experts

    def local_weights(self):
        w = []
        for p in (self.w1, self.w2, self.w3):
            w.append(p.to_local() if hasattr(p, "to_local") else p)
        return w

    def forward(self, x, num_tokens_per_expert):
        """``x`` [rows, D] grouped by (local) expert, ``num_tokens_per_expert`` [E_local]."""
        w1, w2, w3 = self.local_weights()
        mo = _moe_ops()
        if self.quant is not None:
            from torchtitan_b200.ops.quant import quant_grouped_linear as gl

            h = ops.swiglu(gl(x, w1, num_tokens_per_expert, self.quant), gl(x, w3, num_tokens_per_expert, self.quant))
            return gl(h, w2, num_tokens_per_expert, self.quant)
        h = ops.swiglu(mo.grouped_linear(x, w1, num_tokens_per_expert), mo.grouped_linear(x, w3, num_tokens_per_expert))
        return mo.grouped_linear(h, w2, num_tokens_per_expert)

    def init_weights(self, **kwargs) -> None:
        init_std = kwargs.get("init_std")
        assert init_std is not None
        nn.init.trunc_normal_(self.w1, mean=0.0, std=0.02)
        nn.init.trunc_normal_(self.w2, mean=0.0, std=init_std)
        nn.init.trunc_normal_(self.w3, mean=0.0, std=init_std)


class TokenChoiceTopKRouter(Module):
    def __init__(self, *, dim: int, num_experts: int, num_expert_groups: int | None,
                 num_limited_groups: int | None, top_k: int, score_func: Literal["softmax", "sigmoid"],
                 route_norm: bool, route_scale: float, gate_bias: bool, _debug_force_load_balance: bool = False):
        super().__init__()
        self.gate = Linear.Config(bias=gate_bias).build(in_features=dim, out_features=num_experts)
        self.num_experts = num_experts
        self.num_expert_groups = num_expert_groups
        self.num_limited_groups = num_limited_groups
        self.top_k = top_k
        self.score_func = score_func
        self.route_norm = route_norm
        self.route_scale = route_scale
        self._debug_force_load_balance = _debug_force_load_balance

    def forward(self, x, expert_bias=None):
        """``x`` [T, D] -> (top_scores [T,k] fp32, expert indices [T,k], tokens per expert [E])."""
        return _moe_ops().route(
            x, self.gate.weight, self.gate.bias, expert_bias,
            top_k=self.top_k, score_func=self.score_func, route_norm=self.route_norm,
            route_scale=self.route_scale, num_expert_groups=self.num_expert_groups,
            num_limited_groups=self.num_limited_groups, force_balance=self._debug_force_load_balance,
        )

    def init_weights(self, **kwargs) -> None:
        init_std = kwargs.get("init_std")
        assert init_std is not None
        self.gate.init_weights(init_std=init_std)


class TokenReorderer(Module):
    """Orders the T*k (token, slot) pairs by expert (stable)."""

    def __init__(self, *, num_experts: int, top_k: int):
        super().__init__()
        self.num_experts, self.top_k = num_experts, top_k

    def forward(self, top_scores, selected_experts_indices):
        order, counts = _moe_ops().sort_by_expert(selected_experts_indices, self.num_experts)
        return top_scores.reshape(-1)[order], order, counts

    def init_weights(self, **kwargs) -> None:
        return None


class MoE(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        num_experts: int = 8
        num_shared_experts: int = 1
        score_func: Literal["softmax", "sigmoid"] = "sigmoid"
        route_norm: bool = False
        route_scale: float = 1.0
        gate_bias: bool = False
        score_before_experts: bool = True
        top_k: int = 1
        num_expert_groups: int | None = None
        num_limited_groups: int | None = None
        use_grouped_mm: bool = True
        load_balance_coeff: float | None = 1e-3
        aux_loss_coeff: float = 0.0
        """*B200 addition*: weight of a switch-style auxiliary load-balance loss
        ``E * sum_e(fraction_e * mean_prob_e)`` whose gradient is injected at the router; 0 = off."""
        _debug_force_load_balance: bool = False
        hidden_dim: int = 0

    def __init__(self, config: Config, *, dim: int):
        super().__init__()
        E, H = config.num_experts, config.hidden_dim
        self.experts = GroupedExperts(dim=dim, hidden_dim=H, num_experts=E, use_grouped_mm=config.use_grouped_mm)
        self.router = TokenChoiceTopKRouter(
            dim=dim, num_experts=E, num_expert_groups=config.num_expert_groups,
            num_limited_groups=config.num_limited_groups, top_k=config.top_k, score_func=config.score_func,
            route_norm=config.route_norm, route_scale=config.route_scale, gate_bias=config.gate_bias,
            _debug_force_load_balance=config._debug_force_load_balance,
        )
        self.reorderer = TokenReorderer(num_experts=E, top_k=config.top_k)
        self.shared_experts = (
            FeedForward.Config(hidden_dim=H * config.num_shared_experts).build(dim=dim)
            if config.num_shared_experts > 0 else None
        )
        self.score_before_experts = config.score_before_experts
        self.load_balance_coeff = config.load_balance_coeff
        self.aux_loss_coeff = config.aux_loss_coeff
        if self.load_balance_coeff is not None:
            assert self.load_balance_coeff > 0.0
            self.register_buffer("expert_bias", torch.zeros(E, dtype=torch.float32), persistent=True)
        else:
            self.expert_bias = None
        self.register_buffer("tokens_per_expert", torch.zeros(E, dtype=torch.float32), persistent=False)
        # expert tensor parallel (set by parallel/ep.py): the experts' hidden dimension is split over this group, whose
        # ranks hold different sequence shards. The routed path then runs on the group's gathered tokens and its partial
        # sums are reduce-scattered back; the shared experts stay on the local shard.
        self._etp_group = None

    def forward(self, x):
        bs, slen, dim = x.shape
        x = x.reshape(-1, dim)
        if self._etp_group is None:
            out = self._routed(x)
        else:
            from torchtitan_b200.parallel.ep import gather_rows, reduce_scatter_rows

            out = reduce_scatter_rows(self._routed(gather_rows(x, self._etp_group)), self._etp_group)
        if self.shared_experts is not None:
            out = out + self.shared_experts(x)
        return out.reshape(bs, slen, dim)

    def _routed(self, x):
        """Router -> dispatch -> experts -> combine on tokens ``x`` [T, dim]."""
        k = self.router.top_k
        top_scores, idx, counts = self.router(x, self.expert_bias)
        with torch.no_grad():
            self.tokens_per_expert.add_(counts.to(self.tokens_per_expert.dtype))
        if self.aux_loss_coeff > 0.0 and self.training:
            x = _moe_ops().inject_aux_loss(x, self.router.gate.weight, counts, self.aux_loss_coeff, k)
        scores_sorted, order, counts_sorted = self.reorderer(top_scores, idx)

        disp = self.experts.dispatcher
        routed_in, local_counts, ctx = disp.dispatch(x, order, counts_sorted, k)
        if self.score_before_experts:
            routed_in = _moe_ops().scale_rows(routed_in, scores_sorted, disp, ctx)
        routed_out = self.experts(routed_in, local_counts)
        weights = None if self.score_before_experts else top_scores
        fused = disp.combine_to_tokens(routed_out, weights, ctx) if hasattr(disp, "combine_to_tokens") else None
        if fused is not None:
            return fused
        routed_out = disp.combine(routed_out, ctx)
        return _moe_ops().scatter_combine(routed_out, order, weights, x.shape[0], k)

    def init_weights(self, **kwargs) -> None:
        init_std = kwargs.get("init_std")
        buffer_device = kwargs.get("buffer_device")
        assert init_std is not None
        assert isinstance(buffer_device, torch.device)
        self.experts.init_weights(init_std=init_std)
        self.router.init_weights(init_std=init_std)
        if self.shared_experts is not None:
            self.shared_experts.init_weights(init_std=init_std)
        with torch.device(buffer_device):
            self.tokens_per_expert = torch.zeros(self.experts.num_experts, dtype=torch.float32)
            if self.load_balance_coeff is not None:
                self.expert_bias = torch.zeros(self.experts.num_experts, dtype=torch.float32)
