"""Trainer for replica-group fault tolerance.

Parity: torchtitan/experiments/ft/trainer.py:40-596 -- same loop as the base trainer plus: an ``FTManager`` built
right after distributed init; the dataset split over ``dp_degree * group_size`` with this replica's offset; the
fault-tolerant optimizer container (quorum at ``zero_grad``, averaged gradients and commit vote at ``step``);
live-recovery state functions (model + optimizer + scheduler + train state travel to a rejoining replica); optional
semi-synchronous LocalSGD / DiLoCo around the loop; per-replica dataloader checkpoints under ``ft-replica-<id>``.
Here the base ``Trainer`` exposes those points as overridable hooks, so this class only fills them in."""

from __future__ import annotations

from contextlib import nullcontext
from dataclasses import dataclass, field

from torchtitan_b200.tools.logging import logger
from torchtitan_b200.trainer import Trainer

from .config import FaultTolerance
from .diloco import fragment_llm
from .local_sgd import DiLoCo, LocalSGD
from .manager import FTManager
from .optimizer import FTOptimizersContainer


def maybe_semi_sync_training(ft_config: FaultTolerance, ft_manager: FTManager, model, n_layers: int, optimizer,
                             fragment_fn=None):
    """Context manager for ``semi_sync_method`` in {local_sgd, diloco}; a null context otherwise."""
    method = ft_config.semi_sync_method
    if not (ft_config.enable and method is not None):
        return nullcontext()
    assert ft_manager.enabled, "FTManager must be enabled to use semi-sync training."
    logger.info(f"using fragment function to split model: {fragment_fn is not None}")
    if method.lower() == "diloco":
        parts = fragment_fn(model, ft_config, n_layers) if fragment_fn else [model]
        return DiLoCo(ft_manager.manager, parts, optimizer, sync_every=ft_config.sync_steps,
                      should_quantize=ft_config.should_quantize, fragment_sync_delay=ft_config.fragment_sync_delay,
                      fragment_update_alpha=ft_config.fragment_update_alpha)
    if method.lower() == "local_sgd":
        return LocalSGD(ft_manager.manager, model, optimizer, sync_every=ft_config.sync_steps)
    raise ValueError(f"Unknown training method: {method}, only 'diloco' and 'local_sgd' are supported.")


class FaultTolerantTrainer(Trainer):
    @dataclass(kw_only=True, slots=True)
    class Config(Trainer.Config):
        fault_tolerance: FaultTolerance = field(default_factory=FaultTolerance)

    def _post_init_distributed(self) -> None:
        self.ft_manager = FTManager(self.config.fault_tolerance)
        if self.ft_manager.enabled:
            logger.info(f"Fault tolerance enabled: replica {self.ft_manager.replica_id} of {self.ft_manager.group_size}")

    def _dataloader_dp_info(self) -> tuple[int, int]:
        return self.ft_manager.get_dp_info(self.dp_degree, self.dp_rank)

    def _build_optimizers(self):
        ft = self.ft_manager
        opt = FTOptimizersContainer(self.config.optimizer, model_parts=self.model_parts, ft_manager=ft,
                                    use_ft_optimizer=self.config.fault_tolerance.semi_sync_method is None)
        if ft.enabled:
            ft.maybe_set_all_reduce_hook(self.model_parts)
            ft.manager.set_state_dict_fns(self._ft_load_state, self._ft_state)
        return opt

    # ---- live recovery payload ---------------------------------------------------------------------------------
    def _ft_state(self) -> dict:
        from torchtitan_b200.parallel import fsdp

        units = [u for m in self.model_parts for u in fsdp.fsdp_units(m)]
        return {
            "params": [u.shard_flat.detach().cpu() for u in units] if units else
                      [p.detach().cpu() for m in self.model_parts for p in m.parameters()],
            "optim": self.optimizers.state_dict() if hasattr(self, "optimizers") else {},
            "sched": self.lr_schedulers.state_dict() if hasattr(self, "lr_schedulers") else {},
            "train_state": self.state_dict(),
        }

    def _ft_load_state(self, state: dict) -> None:
        import torch

        from torchtitan_b200.parallel import fsdp

        units = [u for m in self.model_parts for u in fsdp.fsdp_units(m)]
        with torch.no_grad():
            if units:
                for u, src in zip(units, state["params"]):
                    u.shard_flat.copy_(src)
                    u.mark_params_updated()
            else:
                ps = [p for m in self.model_parts for p in m.parameters()]
                for p, src in zip(ps, state["params"]):
                    p.copy_(src)
        if state["optim"]:
            self.optimizers.load_state_dict(state["optim"])
        if state["sched"]:
            self.lr_schedulers.load_state_dict(state["sched"])
        self.load_state_dict(state["train_state"])

    def train(self):
        ft_cfg = self.config.fault_tolerance
        n_layers = getattr(self.model_config, "n_layers", 0)
        with maybe_semi_sync_training(ft_cfg, self.ft_manager, self.model_parts[0], n_layers, self.optimizers,
                                      fragment_fn=fragment_llm):
            return super().train()

    def close(self) -> None:
        if getattr(self, "ft_manager", None) is not None and self.ft_manager.enabled:
            self.ft_manager.manager.shutdown()
        super().close()
