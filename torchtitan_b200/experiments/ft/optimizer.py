"""Optimizer container whose ``zero_grad`` opens the step's quorum and whose ``step`` averages gradients over the
live replicas and applies the update only if every replica of the quorum votes to commit.
Parity: torchtitan/experiments/ft/optimizer.py:26-91 (``ft.Optimizer`` semantics; with ``use_ft_optimizer=False``
for semi-sync methods the container behaves like the plain one)."""

from __future__ import annotations

from torchtitan_b200.components.optimizer import OptimizersContainer


class FTOptimizersContainer(OptimizersContainer):
    def __init__(self, config, *, model_parts, ft_manager, use_ft_optimizer: bool = True):
        super().__init__(config, model_parts=model_parts)
        self.ft_manager = ft_manager
        self._use_ft_optimizer = use_ft_optimizer and ft_manager.enabled
        self.cache_state_dict: dict = {}
        self.skipped_steps = 0

    def init_cache_state_dict(self) -> None:
        self.cache_state_dict = super().state_dict()

    def state_dict(self) -> dict:
        return self.cache_state_dict

    def load_state_dict(self, state_dict) -> None:
        super().load_state_dict(state_dict)
        self.init_cache_state_dict()

    def zero_grad(self, *args, **kwargs) -> None:
        if self._use_ft_optimizer:
            self.ft_manager.manager.start_quorum()
        super().zero_grad(*args, **kwargs)

    def step(self, *args, **kwargs) -> None:
        if not self._use_ft_optimizer:
            return super().step(*args, **kwargs)
        self.ft_manager.average_gradients()
        if self.ft_manager.manager.should_commit():
            super().step(*args, **kwargs)
        else:
            self.skipped_steps += 1
