"""``GraphTrainer``: the base trainer whose forward+backward runs from a captured CUDA graph when the plan says so.
Parity: torchtitan/experiments/graph_trainer/trainer.py:14-30 (a thin ``Trainer`` subclass that owns the graph state
and releases it in ``close``)."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from torchtitan_b200.trainer import Trainer

from .configs import GraphTrainerCompileConfig
from .cudagraph import CUDAGraphWrapper
from .passes import build_plan


class GraphTrainer(Trainer):
    @dataclass(kw_only=True, slots=True)
    class Config(Trainer.Config):
        compile: GraphTrainerCompileConfig = field(default_factory=GraphTrainerCompileConfig)

    def __init__(self, config: Config):
        self.plan = build_plan(config.compile.passes, config.compile.joint_passes)
        if self.plan.reshard_after_forward != "default":
            config.parallelism.fsdp_reshard_after_forward = self.plan.reshard_after_forward
        config.parallelism.fsdp_prefetch_depth = max(getattr(config.parallelism, "fsdp_prefetch_depth", 1), self.plan.prefetch_depth)
        if self.plan.bucketing == "auto":
            config.parallelism.fsdp_bucket_bytes = self.plan.bucket_bytes      # consecutive blocks share one FSDP unit
        if self.plan.extra_fsdp_pg:
            config.parallelism.fsdp_extra_process_group = True
        if self.plan.sac_save_ops is not None and config.activation_checkpoint.mode == "none":
            config.activation_checkpoint.mode, config.activation_checkpoint.selective_ac_option = "selective", "op"
        super().__init__(config)
        self._graph_step: CUDAGraphWrapper | None = None

    def forward_backward_step(self, *, input_dict, labels, global_valid_tokens):
        if not (self.plan.cudagraph and self.device.type == "cuda") or self.parallel_dims.pp_enabled:
            return super().forward_backward_step(input_dict=input_dict, labels=labels, global_valid_tokens=global_valid_tokens)
        if self._graph_step is None:
            base = super().forward_backward_step

            def run(inputs, lab, denom):
                return base(input_dict={"input": inputs}, labels=lab, global_valid_tokens=denom)

            self._graph_step = CUDAGraphWrapper(run, warmup=2)
        extra = {k: v for k, v in input_dict.items() if k != "input"}
        if extra:
            raise NotImplementedError("cudagraph capture supports token-only batches")
        return self._graph_step(input_dict["input"], labels, global_valid_tokens)

    def close(self) -> None:
        self._graph_step = None
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        super().close()
