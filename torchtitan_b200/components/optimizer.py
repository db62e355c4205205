"""Optimizer containers.

``OptimizersContainer`` presents one optimizer per model part as a single
``torch.optim.Optimizer`` (so step hooks and LR schedulers work on it) and saves / loads
state through ``get/set_optimizer_state_dict(flatten_optimizer_state_dict=True)``, i.e.
checkpoint keys ``state.<fqn>.exp_avg`` / ``param_groups.<fqn>.lr``.
Parity: torchtitan/components/optimizer.py:37-174. ``OptimizersInBackwardContainer`` steps each
parameter as soon as its gradient is accumulated (:177-225). ``register_moe_load_balancing_hook``
implements auxiliary-loss-free balancing as a step pre-hook (:228-335): all-reduce the per-layer
token histograms over the ``loss`` mesh, ``bias += coeff * sign(mean - count)``, re-centred.

B200 path: with ``implementation="fused"`` on CUDA the parameters that live in FSDP units are
stepped by :class:`ShardAdamW`, which runs one AdamW launch per unit over the unit's flat fp32
shard (master, exp_avg, exp_avg_sq, gradient) and writes the bf16 shadow that the next
all-gather reads in the same pass. The state it exposes per parameter are views of those flat
buffers, so the checkpoint format is unchanged.
"""

from __future__ import annotations

import functools
from dataclasses import dataclass
from typing import Any, Iterator, Literal

import torch
import torch.nn as nn
from torch.distributed.checkpoint.state_dict import (
    StateDictOptions,
    get_optimizer_state_dict,
    set_optimizer_state_dict,
)
from torch.distributed.checkpoint.stateful import Stateful
from torch.distributed.tensor import DTensor, Replicate
from torch.optim import Optimizer

from torchtitan_b200.config.configurable import Configurable

__all__ = [
    "OptimizersContainer",
    "OptimizersInBackwardContainer",
    "ShardAdamW",
    "register_moe_load_balancing_hook",
]


class ShardAdamW(Optimizer):
    """Adam/AdamW over FSDP units' flat shard buffers (plus ordinary tensors as a fallback).

    Update rule is ``torch.optim.AdamW`` (decoupled decay when ``decoupled``; bias-corrected
    moments; eps added after the square root). ``step`` counts are fp32 scalars as in torch so
    state dicts are interchangeable.
    """

    def __init__(self, params, *, units, lr, betas, eps, weight_decay, decoupled=True):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decoupled=decoupled,
                        fused=None, foreach=None, amsgrad=False, maximize=False, capturable=False,
                        differentiable=False)
        super().__init__(params, defaults)
        self.units = list(units)
        self._unit_of: dict[int, tuple] = {}
        for u in self.units:
            u.exp_avg_flat = torch.zeros_like(u.shard_flat)
            u.exp_avg_sq_flat = torch.zeros_like(u.shard_flat)
            u.step_count = 0
            for i, p in enumerate(u.params):
                self._unit_of[id(p.param)] = (u, i)
        self._init_state()
        self.has_loose_params = any(
            id(p) not in self._unit_of for g in self.param_groups for p in g["params"]
        )

    def _wrap_like(self, param, local):
        if isinstance(param, DTensor):
            from torchtitan_b200.parallel.fsdp import _contig_stride, dtensor_over

            return dtensor_over(local, param.device_mesh, param.placements, param.shape, _contig_stride(param.shape))
        return local

    def _init_state(self):
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state[p]
                if id(p) in self._unit_of:
                    u, i = self._unit_of[id(p)]
                    pi = u.params[i]
                    st["step"] = torch.tensor(0.0, dtype=torch.float32)
                    st["exp_avg"] = self._wrap_like(p, u._shard_view(u.exp_avg_flat, pi))
                    st["exp_avg_sq"] = self._wrap_like(p, u._shard_view(u.exp_avg_sq_flat, pi))
                else:
                    st["step"] = torch.tensor(0.0, dtype=torch.float32)
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)

    @torch.no_grad()
    def step(self, closure=None):
        from torchtitan_b200.ops import optim_ops

        group = self.param_groups[0]
        lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
        lr = float(lr)
        for u in self.units:
            if not any(p.param.grad is not None for p in u.params):
                continue
            u.step_count += 1
            optim_ops.adamw_flat(
                u.shard_flat, u.grad_shard_flat, u.exp_avg_flat, u.exp_avg_sq_flat, u.shadow_flat,
                lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd, step=u.step_count,
                decoupled=group["decoupled"], grad_scale=getattr(u, "pending_grad_scale", None),
            )
            u.pending_grad_scale = None
            u.mark_params_updated(shadow_is_fresh=u.shadow_flat is not None)
        for g in self.param_groups:
            for p in g["params"]:
                st = self.state[p]
                if id(p) in self._unit_of:
                    if p.grad is not None:
                        st["step"] += 1
                    continue
                if p.grad is None:
                    continue
                st["step"] += 1
                optim_ops.adamw_flat(
                    p.data.view(-1), p.grad.view(-1), st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1), None,
                    lr=float(g["lr"]), beta1=g["betas"][0], beta2=g["betas"][1], eps=g["eps"],
                    weight_decay=g["weight_decay"], step=int(st["step"].item()), decoupled=g["decoupled"],
                )

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        # loaded tensors are fresh allocations: copy them into the flat buffers and re-point
        for group in self.param_groups:
            for p in group["params"]:
                if id(p) not in self._unit_of:
                    continue
                u, i = self._unit_of[id(p)]
                pi, st = u.params[i], self.state[p]
                for key, flat in (("exp_avg", u.exp_avg_flat), ("exp_avg_sq", u.exp_avg_sq_flat)):
                    view = u._shard_view(flat, pi)
                    loaded = st[key]
                    loaded = loaded._local_tensor if isinstance(loaded, DTensor) else loaded
                    if loaded.data_ptr() != view.data_ptr():
                        view.copy_(loaded)
                    st[key] = self._wrap_like(p, view)
                u.step_count = int(float(st["step"]))


class OptimizersContainer(Optimizer, Stateful, Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        name: str = "AdamW"
        lr: float = 8e-4
        beta1: float = 0.9
        beta2: float = 0.95
        eps: float = 1e-8
        weight_decay: float = 0.1
        implementation: Literal["for-loop", "foreach", "fused"] = "fused"
        """'fused' = this framework's flat-shard kernel on CUDA (torch's fused path is not used);
        'foreach' / 'for-loop' = the corresponding torch.optim implementations."""

    optimizers: list
    model_parts: list[nn.Module]

    @staticmethod
    def _resolve_optimizer_cls(name: str) -> type:
        classes = {"Adam": torch.optim.Adam, "AdamW": torch.optim.AdamW}
        if name not in classes:
            raise NotImplementedError(f"Optimizer {name} not added.")
        return classes[name]

    @staticmethod
    def _build_optimizer_kwargs(config: "OptimizersContainer.Config") -> dict[str, Any]:
        assert config.implementation in ("fused", "foreach", "for-loop")
        return {
            "lr": config.lr,
            "betas": (config.beta1, config.beta2),
            "eps": config.eps,
            "weight_decay": config.weight_decay,
            "fused": config.implementation == "fused",
            "foreach": config.implementation == "foreach",
        }

    @staticmethod
    def _build_one(config, params: list, model: nn.Module):
        kwargs = OptimizersContainer._build_optimizer_kwargs(config)
        cls = OptimizersContainer._resolve_optimizer_cls(config.name)
        on_cuda = any(
            (p._local_tensor if isinstance(p, DTensor) else p).is_cuda for p in params
        )
        if kwargs["fused"] and on_cuda:
            from torchtitan_b200.parallel.fsdp import fsdp_units

            units = [u for u in fsdp_units(model) if u.params and u._materialized]
            return ShardAdamW(params, units=units, lr=config.lr, betas=kwargs["betas"], eps=config.eps,
                              weight_decay=config.weight_decay, decoupled=config.name == "AdamW")
        if kwargs["fused"]:
            kwargs["fused"] = False  # torch's fused kernels are CUDA-only; CPU runs the plain loop
            kwargs["foreach"] = True
        return cls(params, **kwargs)

    def __init__(self, config: Config, *, model_parts: list[nn.Module]) -> None:
        kwargs = self._build_optimizer_kwargs(config)
        all_params: list = []
        self.optimizers = []
        self.model_parts = model_parts
        for model in model_parts:
            params = [p for p in model.parameters() if p.requires_grad]
            self.optimizers.append(self._build_one(config, params, model))
            all_params.extend(params)
        self._validate_length(len(model_parts))
        self._post_init(all_params, kwargs)

    def __iter__(self) -> Iterator:
        return iter(self.optimizers)

    def __len__(self) -> int:
        return len(self.optimizers)

    def step(self, *args, **kwargs) -> None:
        for opt in self.optimizers:
            opt.step(*args, **kwargs)
        self._notify_units()

    def _notify_units(self):
        from torchtitan_b200.parallel.fsdp import fsdp_units

        for model, opt in zip(self.model_parts, self.optimizers):
            if isinstance(opt, ShardAdamW):
                continue
            for u in fsdp_units(model):
                u.mark_params_updated()

    def zero_grad(self, *args, **kwargs) -> None:
        for opt in self.optimizers:
            opt.zero_grad(*args, **kwargs)

    def _outer_sharded_params(self) -> dict:
        from torchtitan_b200.parallel.global_view import is_outer_sharded

        return {n: p for m in self.model_parts for n, p in m.named_parameters(remove_duplicate=False) if is_outer_sharded(p)}

    def state_dict(self) -> dict[str, Any]:
        """Flattened (``state.<fqn>.<name>``, ``param_groups.<fqn>.<option>``). States of tensor- / expert-parallel shards
        appear with the parameter's full logical shape, like the parameters themselves in the model state dict."""
        from torchtitan_b200.parallel.global_view import global_view

        fn = functools.partial(get_optimizer_state_dict, options=StateDictOptions(flatten_optimizer_state_dict=True))
        out = {k: v for sd in map(fn, self.model_parts, self.optimizers) for k, v in sd.items()}
        sharded = self._outer_sharded_params()
        if sharded:
            for k, v in out.items():
                if k.startswith("state.") and torch.is_tensor(v):
                    fqn = k[len("state."):].rsplit(".", 1)[0]
                    if fqn in sharded:
                        out[k] = global_view(sharded[fqn], v)
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        from torchtitan_b200.parallel.global_view import local_of

        sharded = self._outer_sharded_params()
        if sharded:
            # back from full-shape views to tensors laid out like the parameter on this rank
            state_dict = dict(state_dict)
            for k, v in state_dict.items():
                if k.startswith("state.") and torch.is_tensor(v):
                    fqn = k[len("state."):].rsplit(".", 1)[0]
                    p = sharded.get(fqn)
                    if p is not None and v.dim() > 0:
                        local = local_of(v)
                        from torchtitan_b200.parallel.fsdp import dtensor_over

                        state_dict[k] = (dtensor_over(local, p.device_mesh, p.placements, p.shape, p.stride())
                                         if isinstance(p, DTensor) else local)
        fn = functools.partial(
            set_optimizer_state_dict, optim_state_dict=state_dict,
            options=StateDictOptions(flatten_optimizer_state_dict=True),
        )
        list(map(fn, self.model_parts, self.optimizers))

    def _validate_length(self, expected: int) -> None:
        assert expected == len(self.optimizers), (
            "Must pass one optimizer per model part or per param if using OptimizersInBackwardContainer."
        )

    def _post_init(self, all_params, optimizer_kwargs) -> None:
        Optimizer.__init__(self, all_params, optimizer_kwargs)

    def init_cache_state_dict(self) -> None:
        """Hook for fault-tolerant subclasses that cache the state dict; nothing to do here."""


class OptimizersInBackwardContainer(OptimizersContainer):
    """Each parameter has its own optimizer that steps (and clears the gradient) as soon as
    the gradient has been accumulated; ``step``/``zero_grad`` of the container are no-ops."""

    @dataclass(kw_only=True, slots=True)
    class Config(OptimizersContainer.Config):
        pass

    def __init__(self, config: Config, *, model_parts: list[nn.Module]) -> None:
        kwargs = self._build_optimizer_kwargs(config)
        kwargs["fused"], kwargs["foreach"] = False, False
        cls = self._resolve_optimizer_cls(config.name)
        self.model_parts = model_parts
        per_param: dict = {}
        all_params = []
        for model in model_parts:
            for p in model.parameters():
                if p.requires_grad:
                    per_param[p] = cls([p], **kwargs)
                all_params.append(p)

        def hook(param) -> None:
            per_param[param].step()
            per_param[param].zero_grad()

        self._lazy = []
        for model in model_parts:
            for p in model.parameters():
                if p.requires_grad:
                    try:
                        p.register_post_accumulate_grad_hook(hook)
                    except RuntimeError:
                        self._lazy.append(p)  # gradients assigned outside autograd (sharded params)
        self._per_param = per_param
        self.optimizers = list(per_param.values())
        self._validate_length(sum(len(list(m.parameters())) for m in model_parts))
        self._post_init(all_params, kwargs)

    def step(self) -> None:
        # sharded parameters receive .grad from the FSDP unit, not from autograd: step them now
        for p, opt in self._per_param.items():
            if p.grad is not None:
                opt.step()
                opt.zero_grad()
        self._notify_units()

    def zero_grad(self) -> None:
        pass


def _moe_blocks(model_parts):
    for part in model_parts:
        layers = part.get_submodule("layers")
        for block in layers.values():
            if getattr(block, "moe_enabled", False):
                yield block


def register_moe_load_balancing_hook(optimizers: OptimizersContainer, model_parts: list[nn.Module], parallel_dims) -> None:
    blocks = list(_moe_blocks(model_parts))
    if not blocks or not blocks[0].moe.load_balance_coeff:
        return

    def recomputed(block) -> bool:
        return bool(getattr(block, "_ac_recomputes_forward", False))

    def update(*_a, **_k):
        blocks = list(_moe_blocks(model_parts))
        counts = []
        for b in blocks:
            if b.moe.load_balance_coeff is None:
                return
            t = b.moe.tokens_per_expert
            counts.append(t // 2 if recomputed(b) else t)
        by_layer = torch.vstack(counts)
        loss_mesh = parallel_dims.get_optional_mesh("loss")
        if loss_mesh is not None:
            if isinstance(by_layer, DTensor):
                by_layer = by_layer.redistribute(placements=[Replicate()] * by_layer.device_mesh.ndim)
            else:
                torch.distributed.all_reduce(by_layer, group=loss_mesh.get_group())
        with torch.no_grad():
            for i, b in enumerate(blocks):
                t = by_layer[i].float()
                delta = b.moe.load_balance_coeff * torch.sign(t.mean() - t)
                b.moe.expert_bias.add_(delta - delta.mean())
                b.moe.tokens_per_expert.zero_()

    optimizers.register_step_pre_hook(update)
