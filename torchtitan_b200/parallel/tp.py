"""Tensor parallel with sequence parallel and loss parallel for decoder models.

Same plan as torchtitan/models/llama3/parallelize.py:175-268 (and the Qwen3 variant,
torchtitan/models/qwen3/parallelize.py:201-308): embeddings are vocab-sharded and emit
sequence-sharded activations; norms work on sequence shards; before attention and the FFN the
sequence is all-gathered, ``wq/wk/wv/w1/w3`` are column-parallel (heads / hidden split), ``wo/w2``
are row-parallel followed by a reduce-scatter back to sequence shards; the output projection is
column-parallel over the vocabulary and the loss is computed on vocab shards (loss parallel,
torchtitan/distributed/utils.py:216-225) unless disabled.

Built differently: no DTensor dispatch on the hot path. Parameters become plain local shards
tagged with ``_tp_placement`` (so FSDP shards them further and checkpoints can describe them),
and the four collectives are explicit autograd functions. With
``parallelism.enable_async_tensor_parallel`` on CUDA the gather->GEMM and GEMM->reduce-scatter
pairs run through the fused kernels of ``parallel/async_tp.py`` instead of collective + GEMM.
"""

from __future__ import annotations

import functools

import torch
import torch.distributed as dist
import torch.nn as nn

from torchtitan_b200.tools.logging import logger

__all__ = ["apply_tp_to_decoder", "finalize_tp", "LOSS_PARALLEL", "vocab_parallel_cross_entropy_sum", "sync_replicated_params"]


class _LossParallel:
    enabled = False
    group = None


LOSS_PARALLEL = _LossParallel()


# ---------------------------------------------------------------------------- collectives
class _AllGatherSeq(torch.autograd.Function):
    """[B, S/tp, D] -> [B, S, D]; backward = reduce-scatter on the sequence dimension."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = dist.get_world_size(group)
        xt = x.transpose(0, 1).contiguous()  # [S/tp, B, D]: gather along dim 0
        out = torch.empty((W * xt.shape[0],) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, xt, group=group)
        return out.transpose(0, 1).contiguous()

    @staticmethod
    def backward(ctx, g):
        W = dist.get_world_size(ctx.group)
        gt = g.transpose(0, 1).contiguous()
        out = torch.empty((gt.shape[0] // W,) + tuple(gt.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, gt, group=ctx.group)
        return out.transpose(0, 1).contiguous(), None


class _ReduceScatterSeq(torch.autograd.Function):
    """partial [B, S, D] -> summed [B, S/tp, D]; backward = all-gather."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = dist.get_world_size(group)
        xt = x.transpose(0, 1).contiguous()
        out = torch.empty((xt.shape[0] // W,) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, xt, group=group)
        return out.transpose(0, 1).contiguous()

    @staticmethod
    def backward(ctx, g):
        W = dist.get_world_size(ctx.group)
        gt = g.transpose(0, 1).contiguous()
        out = torch.empty((W * gt.shape[0],) + tuple(gt.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, gt, group=ctx.group)
        return out.transpose(0, 1).contiguous(), None


class _AllGatherLast(torch.autograd.Function):
    """[.., V/tp] -> [.., V]; backward = slice."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group, ctx.n = group, x.shape[-1]
        W = dist.get_world_size(group)
        parts = [torch.empty_like(x) for _ in range(W)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        r = dist.get_rank(ctx.group)
        return g[..., r * ctx.n : (r + 1) * ctx.n].contiguous(), None


class _AllReduceSum(torch.autograd.Function):
    """Sum over the group; the gradient passes through unchanged (every rank holds the full gradient)."""

    @staticmethod
    def forward(ctx, x, group):
        out = x.contiguous().clone()
        dist.all_reduce(out, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return g, None


def all_gather_seq(x, group):
    return _AllGatherSeq.apply(x, group)


def reduce_scatter_seq(x, group):
    return _ReduceScatterSeq.apply(x, group)


# ---------------------------------------------------------------------------- loss parallel
class _VocabParallelCE(torch.autograd.Function):
    """Sum of token cross-entropies from vocabulary-sharded logits (fp32 math).

    Three small all-reduces over the TP group per call: row max, sum-exp, target logit
    (the message sizes of torchtitan's loss-parallel path)."""

    @staticmethod
    def forward(ctx, logits, labels, group, ignore_index):
        W, r = dist.get_world_size(group), dist.get_rank(group)
        Vl = logits.shape[-1]
        lg = logits.reshape(-1, Vl).float()
        lab = labels.reshape(-1)
        m = lg.max(dim=-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        ex = torch.exp(lg - m[:, None])
        se = ex.sum(-1)
        dist.all_reduce(se, group=group)
        local = lab - r * Vl
        mine = (local >= 0) & (local < Vl) & (lab != ignore_index)
        tgt = torch.zeros_like(m)
        idx = local.clamp(0, Vl - 1)
        tgt = torch.where(mine, lg.gather(1, idx[:, None]).squeeze(1), tgt)
        dist.all_reduce(tgt, group=group)
        valid = lab != ignore_index
        loss_rows = torch.where(valid, torch.log(se) + m - tgt, torch.zeros_like(m))
        ctx.save_for_backward(ex, se, idx, mine, valid)
        ctx.shape, ctx.dtype = logits.shape, logits.dtype
        return loss_rows.sum()

    @staticmethod
    def backward(ctx, g):
        ex, se, idx, mine, valid = ctx.saved_tensors
        p = ex / se[:, None]
        p[torch.arange(p.shape[0], device=p.device)[mine], idx[mine]] -= 1.0
        p = p * valid[:, None].to(p.dtype) * g
        return p.to(ctx.dtype).view(ctx.shape), None, None, None


def vocab_parallel_cross_entropy_sum(logits, labels, group, ignore_index: int = -100):
    return _VocabParallelCE.apply(logits, labels, group, ignore_index)


# ---------------------------------------------------------------------------- parameter sharding
# Specs are kept on the *module* (``mod._tp_specs[name]``) because ``nn.Module.to_empty`` may
# replace or swap Parameter objects and drop Python attributes; ``finalize_tp`` re-applies them.
def _tag(p, spec) -> None:
    p._tp_placement = spec["placement"]
    p._tp_group, p._tp_mesh = spec["group"], spec["mesh"]
    p._tp_full_shape = spec.get("full_shape")
    # every sharding applied to the full tensor, outermost first: (dim, mesh) -- what a checkpoint view needs
    chain, s = [], spec
    while s is not None:
        if s["placement"][0] == "shard":
            chain.append((s["placement"][1], s["mesh"]))
        s = s.get("outer")
    p._tp_chain = tuple(reversed(chain))
    if spec["placement"][0] == "shard":
        # its squared norm is a partial sum over the TP group (over several groups for 2-D expert shards)
        p._extra_norm_groups = tuple(spec.get("norm_groups") or (spec["group"],))


def _shard_param(mod: nn.Module, name: str, dim: int, rank: int, world: int, group, mesh) -> None:
    p = getattr(mod, name)
    if p is None:
        return
    assert p.shape[dim] % world == 0, f"{name}: dim {dim} of size {p.shape[dim]} not divisible by tp={world}"
    n = p.shape[dim] // world
    if p.device.type == "meta":
        shape = list(p.shape)
        shape[dim] = n
        local = torch.empty(shape, dtype=p.dtype, device="meta")
    else:
        local = p.detach().narrow(dim, rank * n, n).clone()
    newp = nn.Parameter(local, requires_grad=p.requires_grad)
    spec = {"placement": ("shard", dim), "group": group, "mesh": mesh, "full_shape": tuple(p.shape)}
    mod.__dict__.setdefault("_tp_specs", {})[name] = spec
    _tag(newp, spec)
    mod._parameters[name] = newp


class _ScaleFwd(torch.autograd.Function):
    """``bias / W`` in forward, identity in backward."""

    @staticmethod
    def forward(ctx, b, W):
        return b / W

    @staticmethod
    def backward(ctx, g):
        return g, None


def _mark_replicated(mod: nn.Module, group, mesh) -> None:
    """Replicated parameters that only see this rank's sequence shard: their gradients are partial
    sums and must be all-reduced over the TP group (a tensor hook, or the FSDP unit when it owns them)."""
    for name, p in mod._parameters.items():
        if p is None or name in mod.__dict__.get("_tp_specs", {}):
            continue
        spec = {"placement": ("replicate", None), "group": group, "mesh": mesh, "full_shape": tuple(p.shape)}
        mod.__dict__.setdefault("_tp_specs", {})[name] = spec
        _tag(p, spec)


def _grad_allreduce_hook(group):
    def hook(grad):
        grad = grad.contiguous()
        dist.all_reduce(grad, group=group)
        return grad

    return hook


def finalize_tp(model: nn.Module) -> None:
    """Call after ``to_empty`` + ``init_weights``: re-tag parameters from the module-level specs,
    install gradient all-reduce hooks on replicated leaf parameters that no FSDP unit owns, and
    make replicated parameters identical across the TP group (ranks initialise with distinct seeds
    so that *sharded* parameters differ)."""
    any_tp = False
    for mod in model.modules():
        specs = mod.__dict__.get("_tp_specs")
        if not specs:
            continue
        any_tp = True
        for name, spec in specs.items():
            p = mod._parameters.get(name)
            if p is None:
                continue
            _tag(p, spec)
            owned = getattr(p, "_tt_unit", None) is not None
            if spec["placement"][0] == "replicate":
                t = p._local_tensor if hasattr(p, "_local_tensor") else p.data
                if t.device.type != "meta":
                    dist.broadcast(t, src=dist.get_global_rank(spec["group"], 0), group=spec["group"])
                if not owned and p.requires_grad and not mod.__dict__.get("_tp_hooked_" + name):
                    mod.__dict__["_tp_hooked_" + name] = True
                    p.register_hook(_grad_allreduce_hook(spec["group"]))
    if any_tp:
        from .fsdp import fsdp_units

        for u in fsdp_units(model):
            u.mark_params_updated()


def sync_replicated_params(model: nn.Module) -> None:
    finalize_tp(model)


# ---------------------------------------------------------------------------- module surgery
def _wrap(module: nn.Module, fn):
    inner = module.forward

    @functools.wraps(inner)
    def forward(*a, **k):
        return fn(inner, *a, **k)

    module.forward = forward


def apply_tp_to_decoder(model: nn.Module, tp_mesh, *, loss_parallel: bool = True, async_tp: bool = False,
                        cp_enabled: bool = False, enable_float8_tensorwise_tp: bool = False,
                        sequence_parallel: bool = True) -> nn.Module:
    group = tp_mesh.get_group()
    if sequence_parallel:
        _gather, _scatter = all_gather_seq, reduce_scatter_seq
    else:
        # inference plan (generation scripts): activations stay replicated, partial sums are all-reduced
        _gather, _scatter = (lambda x, g: x), (lambda x, g: _AllReduceSum.apply(x, g))
    W, r = tp_mesh.size(), tp_mesh.get_local_rank()
    fused = None
    if async_tp and torch.cuda.is_available():
        try:
            from .async_tp import AsyncTP

            fused = AsyncTP.maybe_create(tp_mesh)
        except ImportError:
            fused = None
        logger.info(f"Async TP: {'fused gather-GEMM / GEMM-reduce-scatter kernels' if fused else 'unavailable, using collectives'}")

    # ---- embedding: vocab-parallel lookup, output reduce-scattered to sequence shards -----------
    emb = getattr(model, "tok_embeddings", None)
    if emb is not None:
        _shard_param(emb, "weight", 0, r, W, group, tp_mesh)
        Vl = emb.weight.shape[0]

        def emb_forward(inner, tokens):
            lo = r * Vl
            local = tokens - lo
            ok = (local >= 0) & (local < Vl)
            out = torch.nn.functional.embedding(local.clamp(0, Vl - 1), emb.weight)
            out = out * ok.unsqueeze(-1).to(out.dtype)
            return _scatter(out, group)

        _wrap(emb, emb_forward)

    # ---- blocks --------------------------------------------------------------------------------------
    for block in model.layers.values():
        att = block.attention
        if hasattr(att, "wkv_b"):
            # multi-head latent attention: the per-head up-projections are column-parallel, the shared low-rank
            # down-projections and their norms stay replicated
            col = ("wq", "wq_b", "wkv_b")
            for nm in ("wq_a", "wkv_a", "q_norm", "kv_norm"):
                if getattr(att, nm, None) is not None:
                    _mark_replicated(getattr(att, nm), group, tp_mesh)
        else:
            col = ("wq", "wk", "wv")
        for name in col:
            lin = getattr(att, name, None)
            if lin is None:
                continue
            _shard_param(lin, "weight", 0, r, W, group, tp_mesh)
            if lin.bias is not None:
                _shard_param(lin, "bias", 0, r, W, group, tp_mesh)
        _shard_param(att.wo, "weight", 1, r, W, group, tp_mesh)
        if att.wo.bias is not None:
            # a row-parallel bias must enter the cross-rank sum exactly once: every rank adds bias / W. Its
            # gradient sees the full (all-gathered) output gradient on every rank, so it needs no reduction.
            from torchtitan_b200 import ops as _ops

            _wrap(att.wo, lambda inner, x, _lin=att.wo: _ops.linear(x, _lin.weight, None) + _ScaleFwd.apply(_lin.bias, W))
        if getattr(att, "sinks", None) is not None:
            _shard_param(att, "sinks", 0, r, W, group, tp_mesh)
        for nm in ("q_norm", "k_norm"):
            if getattr(att, nm, None) is not None:
                _mark_replicated(getattr(att, nm), group, tp_mesh)
        if fused is not None:
            fused.attach_attention(att)

        def att_forward(inner, x, *a, _att=att, **k):
            atp = _att.__dict__.get("_async_tp")
            if atp is not None and atp.attention_supported(_att, x):
                _att.__dict__["_fused_tp_call"] = atp
                try:
                    return inner(x, *a, **k)             # gathers and reduce-scatters inside its GEMMs
                finally:
                    _att.__dict__.pop("_fused_tp_call", None)
            return _scatter(inner(_gather(x, group), *a, **k), group)

        _wrap(att, att_forward)
        ff = getattr(block, "feed_forward", None)
        if ff is not None and not getattr(block, "moe_enabled", False):
            _shard_param(ff.w1, "weight", 0, r, W, group, tp_mesh)
            _shard_param(ff.w3, "weight", 0, r, W, group, tp_mesh)
            _shard_param(ff.w2, "weight", 1, r, W, group, tp_mesh)
            if fused is not None:
                fused.attach_ffn(ff)

                def ffn_forward(inner, x, _ff=ff):
                    if _ff._async_tp.supported(x, _ff.w1.weight):
                        from .async_tp import fused_ffn_forward

                        y, scattered = fused_ffn_forward(_ff, x, group)
                        return y if scattered else _scatter(y, group)
                    return _scatter(inner(_gather(x, group)), group)

                _wrap(ff, ffn_forward)
            else:
                _wrap(ff, lambda inner, x, *a, **k: _scatter(inner(_gather(x, group), *a, **k), group))
        for nm in ("attention_norm", "ffn_norm"):
            if getattr(block, nm, None) is not None:
                _mark_replicated(getattr(block, nm), group, tp_mesh)
        block._tp_group = group  # MoE blocks are finished by parallel/ep.py

    # ---- final norm + output ---------------------------------------------------------------------------
    if getattr(model, "norm", None) is not None:
        _mark_replicated(model.norm, group, tp_mesh)
    out = getattr(model, "output", None)
    if out is not None:
        _shard_param(out, "weight", 0, r, W, group, tp_mesh)
        LOSS_PARALLEL.group = group

        def out_forward(inner, x):
            y = inner(_gather(x, group))  # [B, S, V/tp]
            if loss_parallel:
                y._tp_vocab_sharded = group  # consumed by the loss (see components/loss.py)
                return y
            return _AllGatherLast.apply(y, group)

        _wrap(out, out_forward)
    elif getattr(model, "norm", None) is None:
        pass
    # pipeline stages without an output layer return sequence shards; the next stage expects them too
    model._tp_group = group
    logger.info(f"Applied Tensor Parallelism (degree {W}, sequence parallel, loss parallel {loss_parallel})")
    return model
