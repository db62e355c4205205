"""Activation checkpointing: ``full``, ``selective`` by layer frequency, ``selective`` per op, ``memory_budget``.

Parity: torchtitan/distributed/activation_checkpoint.py:27-260. Per-op policy (:105-135): ops on
the save list are kept, except that only every *second* matmul is kept; matmuls whose weight
shape matches a Linear named in ``per_op_sac_force_recompute_mm_shapes_by_fqns`` are always
recomputed (and do not advance the counter); device-to-host copies are always kept. The save list
(torchtitan/models/llama3/parallelize.py:44-60) contains matmuls, attention outputs, max
reductions and collective results (reduce-scatter / all-to-all outputs are saved rather than
re-communicated).

Built differently: a block's ``forward`` is wrapped in place (no wrapper module, so parameter
names do not change), and the policy recognises both the ATen ops of the CPU path and this
framework's ``tt_b200::*`` custom ops of the CUDA path.
"""

from __future__ import annotations

import functools
import os
from collections import defaultdict

import torch
import torch.nn as nn
from torch.utils.checkpoint import CheckpointPolicy, checkpoint, create_selective_checkpoint_contexts

from torchtitan_b200.tools.logging import logger

_layer_sac_count = 0


def _resolve(names):
    out = set()
    for ns, name in names:
        pkt = getattr(getattr(torch.ops, ns, None), name, None)
        if pkt is None:
            continue
        try:
            out.add(pkt.default)
        except AttributeError:
            pass
    return out


def _ensure_custom_ops_registered() -> None:
    """The ``tt_b200::*`` ops are defined when ``ops.cuda_ops`` is imported; do that before their
    names are looked up so the policy can recognise them."""
    if torch.cuda.is_available():
        from torchtitan_b200.ops import cuda_ops  # noqa: F401


def default_op_sac_save_list() -> set:
    """Compute-heavy ops whose outputs are kept for backward."""
    _ensure_custom_ops_registered()
    aten = torch.ops.aten
    ops = {
        aten.mm.default, aten.linear.default, aten.addmm.default, aten.bmm.default,
        aten._scaled_dot_product_efficient_attention.default,
        aten._scaled_dot_product_flash_attention.default,
        aten._scaled_dot_product_cudnn_attention.default,
        aten._scaled_dot_product_attention_math.default,
        aten._scaled_dot_product_flash_attention_for_cpu.default,
        aten.max.default,
    }
    ops |= _resolve([
        ("_c10d_functional", "reduce_scatter_tensor"), ("_c10d_functional", "all_to_all_single"),
        ("tt_b200", "gemm"), ("tt_b200", "gemm_res"), ("tt_b200", "mx_mm"), ("tt_b200", "attention_fwd"),
        ("tt_b200", "grouped_gemm"),
        ("tt_b200", "tp_reduce_scatter"), ("tt_b200", "ep_all_to_all"),
    ])
    return ops


def _mm_ops() -> set:
    _ensure_custom_ops_registered()
    aten = torch.ops.aten
    return {aten.mm.default, aten.linear.default} | _resolve([("tt_b200", "gemm"), ("tt_b200", "gemm_res"), ("tt_b200", "mx_mm")])


def _wrap_forward(module: nn.Module, ac_config, context_fn=None) -> nn.Module:
    inner = module.forward
    kwargs = dict(use_reentrant=False, preserve_rng_state=ac_config.preserve_rng_state,
                  determinism_check=ac_config.determinism_check, debug=ac_config.debug)
    if context_fn is not None:
        kwargs["context_fn"] = context_fn

    @functools.wraps(inner)
    def forward(*args, **kw):
        if not torch.is_grad_enabled():
            return inner(*args, **kw)
        prev = torch.utils.checkpoint._enable_checkpoint_early_stop if hasattr(torch.utils.checkpoint, "_enable_checkpoint_early_stop") else None
        with torch.utils.checkpoint.set_checkpoint_early_stop(ac_config.early_stop):
            return checkpoint(inner, *args, **kwargs, **kw)

    module.forward = forward
    module._ac_recomputes_forward = True
    return module


def _apply_full_ac(module, ac_config):
    return _wrap_forward(module, ac_config)


def _apply_layer_sac(module, ac_config):
    global _layer_sac_count
    _layer_sac_count += 1
    freq = int(ac_config.selective_ac_option)
    if not freq or _layer_sac_count % freq == 0:
        return _wrap_forward(module, ac_config)
    return module


_AUTO_KEEP_ALL: bool | None = None


def _auto_keep_all_mm() -> bool:
    """Decided once, at the first checkpointed forward (parameters, gradients and optimizer state are resident by then):
    keep every matmul output when more than 35 % of the device memory is still free."""
    global _AUTO_KEEP_ALL
    if _AUTO_KEEP_ALL is None:
        if torch.cuda.is_available():
            free, total = torch.cuda.mem_get_info()
            reusable = torch.cuda.memory_reserved() - torch.cuda.memory_allocated()   # cached blocks count as free
            _AUTO_KEEP_ALL = (free + reusable) > 0.35 * total
        else:
            _AUTO_KEEP_ALL = False
        logger.info(f"per-op SAC matmul policy (auto): {'all matmul outputs kept' if _AUTO_KEEP_ALL else 'every second matmul kept'}")
    return _AUTO_KEEP_ALL


def _apply_op_sac(module, ac_config, *, base_fqn=None, op_sac_save_list=None):
    save_list = op_sac_save_list or default_op_sac_save_list()
    mm_ops = _mm_ops()
    force = set()
    for fqn, sub in module.named_modules():
        full = f"{base_fqn}.{fqn}" if base_fqn is not None else fqn
        if not any(f in full for f in ac_config.per_op_sac_force_recompute_mm_shapes_by_fqns):
            continue
        if not isinstance(sub, nn.Linear):
            raise ValueError(f"per_op_sac_force_recompute_mm_shapes_by_fqns expected to match a nn.Linear, but got: {sub}")
        out_f, in_f = sub.weight.shape
        force.add((in_f, out_f))

    mm_mode = getattr(ac_config, "per_op_sac_mm_policy", "every_second")

    def keep_all_mm() -> bool:
        if mm_mode != "auto":
            return mm_mode == "all"
        return _auto_keep_all_mm()

    def make_policy(meta):
        keep_all = keep_all_mm()

        def policy(ctx, func, *args, **kwargs):
            if (func == torch.ops.aten._to_copy.default and "cuda" in str(args[0].device)
                    and str(kwargs.get("device", "")) == "cpu"):
                return CheckpointPolicy.MUST_SAVE
            key = "recompute_mm_count" if ctx.is_recompute else "forward_mm_count"
            if func in mm_ops:
                w = args[1].shape
                if func != torch.ops.aten.mm.default:  # linear-style ops carry the weight as [out, in]
                    w = torch.Size((w[1], w[0]))
                if tuple(w) in force:
                    return CheckpointPolicy.PREFER_RECOMPUTE
                meta[key] += 1
            keep = func in save_list and not (func in mm_ops and not keep_all and meta[key] % 2 == 0)
            return CheckpointPolicy.MUST_SAVE if keep else CheckpointPolicy.PREFER_RECOMPUTE

        return policy

    def context_fn():
        return create_selective_checkpoint_contexts(make_policy(defaultdict(int)))

    return _wrap_forward(module, ac_config, context_fn=context_fn)


def _apply_ac_to_transformer_block(module, ac_config, *, base_fqn=None, model_compile_enabled=False, op_sac_save_list=None):
    if ac_config.mode not in ("full", "selective"):
        raise ValueError(f"Invalid AC mode: {ac_config.mode}. Valid modes: ('full', 'selective')")
    if ac_config.mode == "full":
        return _apply_full_ac(module, ac_config)
    opt = ac_config.selective_ac_option
    if opt == "op":
        return _apply_op_sac(module, ac_config, base_fqn=base_fqn, op_sac_save_list=op_sac_save_list)
    if opt.isdigit():
        return _apply_layer_sac(module, ac_config)
    raise ValueError(
        f"Invalid selective AC option: {opt}. Valid options: 'op' or a positive int representing layer frequency"
    )


# Plans a block can take under ``memory_budget``, from cheapest in memory to cheapest in recompute: (name, share of the
# block's no-checkpoint activation bytes that stays resident, share of the block's forward that backward runs again).
# The shares are nominal figures for a dense pre-norm transformer block in bf16 (block input only / matmul outputs,
# attention output and every second matmul / all matmul outputs / everything); they order the plans and set the mix, and
# the planner needs no trace of the model.
_BUDGET_LADDER = (("full", 0.04, 1.0), ("op_every_second", 0.40, 0.55), ("op_all", 0.65, 0.15), ("none", 1.0, 0.0))


def plan_memory_budget(n_blocks: int, budget: float) -> list[str]:
    """One plan name per block such that the mean resident share is the largest reachable value <= ``budget``.

    The reference hands ``memory_budget`` to the partitioner of its tracing compiler, which solves a knapsack over the
    ops of the traced graph (torchtitan/distributed/activation_checkpoint.py:216-230). Without a tracer the same knob is
    served per block: the two neighbouring plans of the ladder around ``budget`` are mixed, the costlier-in-memory one
    on as many blocks as the budget allows, spread evenly over depth so that pipeline stages get the same mix."""
    if not 0.0 <= budget <= 1.0:
        raise ValueError(f"activation_checkpoint.memory_budget must be in [0, 1], got {budget}")
    shares = [x[1] for x in _BUDGET_LADDER]
    if budget <= shares[0]:
        return [_BUDGET_LADDER[0][0]] * n_blocks
    hi = next(i for i, sh in enumerate(shares) if sh >= budget)
    lo = hi - 1
    n_hi = int((budget - shares[lo]) / (shares[hi] - shares[lo]) * n_blocks + 1e-9)
    plans = [_BUDGET_LADDER[lo][0]] * n_blocks
    for k in range(n_hi):                                   # evenly spaced positions
        plans[int((k + 0.5) * n_blocks / n_hi)] = _BUDGET_LADDER[hi][0]
    return plans


def _apply_memory_budget(model, ac_config, *, op_sac_save_list=None, base_folder: str = "") -> None:
    import copy

    blocks = list(model.get_submodule("layers").named_children())
    plans = plan_memory_budget(len(blocks), float(ac_config.memory_budget))

    def variant(**kw):
        c = copy.copy(ac_config)
        for k, v in kw.items():
            setattr(c, k, v)
        return c

    for (layer_id, block), plan in zip(blocks, plans):
        if plan == "full":
            _apply_full_ac(block, ac_config)
        elif plan in ("op_every_second", "op_all"):
            cfg = variant(mode="selective", selective_ac_option="op",
                          per_op_sac_mm_policy="all" if plan == "op_all" else "every_second")
            _apply_op_sac(block, cfg, base_fqn=f"layers.{layer_id}", op_sac_save_list=op_sac_save_list)
    counts = {name: plans.count(name) for name, _, _ in _BUDGET_LADDER if name in plans}
    logger.info(f"Applied memory_budget={ac_config.memory_budget} activation checkpointing: {counts}")
    if ac_config.visualize_memory_budget_pareto and base_folder:
        # the trade-off curve of the ladder for this depth: budget -> resident share, recomputed share of the forward
        os.makedirs(base_folder, exist_ok=True)
        path = os.path.join(base_folder, "memory_budget_pareto.csv")
        share = {n: (m, r) for n, m, r in _BUDGET_LADDER}
        with open(path, "w") as f:
            f.write("budget,resident_share,recompute_share\n")
            for i in range(21):
                pl = plan_memory_budget(len(blocks), i / 20)
                f.write(f"{i / 20:.2f},{sum(share[x][0] for x in pl) / len(pl):.4f},{sum(share[x][1] for x in pl) / len(pl):.4f}\n")
        logger.info(f"memory-budget trade-off table written to {path}")


def apply_ac(model: nn.Module, ac_config, *, model_compile_enabled: bool = False, op_sac_save_list=None,
             base_folder: str = "") -> None:
    if ac_config.mode == "memory_budget":
        _apply_memory_budget(model, ac_config, op_sac_save_list=op_sac_save_list, base_folder=base_folder)
        return
    layers = model.get_submodule("layers")
    for layer_id, block in layers.named_children():
        _apply_ac_to_transformer_block(
            block, ac_config, base_fqn=f"layers.{layer_id}", model_compile_enabled=model_compile_enabled,
            op_sac_save_list=op_sac_save_list,
        )
    logger.info(f"Applied {ac_config.mode} activation checkpointing to the model")
