"""The construction half of the trainer as a reusable object.

Field names follow torchtitan/experiments/forge/engine.py:35-120: besides the usual trainer attributes the engine
exposes ``dp_degree / dp_rank`` (for the caller's own dataloader), ``model_config``, ``num_flops_per_token``,
``model_param_count`` and ``global_batch_size``. No dataloader, tokenizer, metrics processor or validator is created."""

from __future__ import annotations

import os
from dataclasses import asdict, dataclass, field
from typing import Any

import torch
import torch.distributed as dist
from torch.distributed.checkpoint.stateful import Stateful

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import (
    TORCH_DTYPE_MAP, ActivationCheckpointConfig, CommConfig, CompileConfig, DebugConfig, ParallelismConfig, TrainingConfig,
)
from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.parallel import ParallelDims
from torchtitan_b200.parallel import utils as dist_utils
from torchtitan_b200.protocols.model_converter import ModelConvertersContainer
from torchtitan_b200.protocols.model_spec import ModelSpec
from torchtitan_b200.tools import utils
from torchtitan_b200.tools.logging import logger


class ForgeEngine(Stateful, Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        hf_assets_path: str = "./tests/assets/tokenizer"
        dump_folder: str = "./outputs"
        model_spec: ModelSpec | None = None
        optimizer: OptimizersContainer.Config = field(default_factory=OptimizersContainer.Config)
        lr_scheduler: LRSchedulersContainer.Config = field(default_factory=LRSchedulersContainer.Config)
        training: TrainingConfig = field(default_factory=TrainingConfig)
        parallelism: ParallelismConfig = field(default_factory=ParallelismConfig)
        checkpoint: CheckpointManager.Config = field(default_factory=CheckpointManager.Config)
        activation_checkpoint: ActivationCheckpointConfig = field(default_factory=ActivationCheckpointConfig)
        compile: CompileConfig = field(default_factory=CompileConfig)
        model_converters: ModelConvertersContainer.Config = field(default_factory=ModelConvertersContainer.Config)
        comm: CommConfig = field(default_factory=CommConfig)
        debug: DebugConfig = field(default_factory=DebugConfig)

        def to_dict(self) -> dict[str, Any]:
            d = {k: v for k, v in asdict(self).items() if k != "model_spec"}
            d["model_spec"] = None if self.model_spec is None else {"name": self.model_spec.name, "flavor": self.model_spec.flavor}
            return d

    def __init__(self, config: Config):
        self.config = config
        assert config.model_spec is not None
        self.train_spec = spec = config.model_spec
        dev_type = utils.device_type
        self.device = torch.device(f"{dev_type}:{int(os.environ.get('LOCAL_RANK', 0))}") if dev_type == "cuda" else torch.device("cpu")
        if dev_type == "cuda":
            torch.cuda.set_device(self.device)
        world = dist_utils.init_distributed(config.comm, enable_cpu_backend=config.training.enable_cpu_offload,
                                            base_folder=config.dump_folder)
        p = config.parallelism
        self.parallel_dims = pd = ParallelDims(
            dp_shard=p.data_parallel_shard_degree, dp_replicate=p.data_parallel_replicate_degree, cp=p.context_parallel_degree,
            tp=p.tensor_parallel_degree, pp=p.pipeline_parallel_degree, ep=p.expert_parallel_degree,
            etp=p.expert_tensor_parallel_degree, world_size=world,
        )
        if pd.dp_enabled:
            self.dp_degree, self.dp_rank = pd.dim_size("batch"), pd.coordinate("batch", dist.get_rank())
        else:
            self.dp_degree, self.dp_rank = 1, 0
        self.gc_handler = utils.GarbageCollection(gc_freq=config.training.gc_freq, debug=config.training.gc_debug)
        seed_dims = ["pp"] + (["tp"] if pd.tp_enabled else []) + (["ep"] if pd.ep_enabled else [])
        dist_utils.set_determinism(pd, self.device, config.debug, distinct_seed_mesh_dims=seed_dims)

        self.model_config = model_config = spec.model
        model_config.update_from_config(trainer_config=config)
        with torch.device("meta"), utils.set_default_dtype(TORCH_DTYPE_MAP[config.training.dtype]):
            model = model_config.build()
        converters = config.model_converters.build(parallel_dims=pd, model_compile_enabled=config.compile.enable)
        converters.convert(model)
        self.model_param_count, self.num_flops_per_token = model_config.get_nparams_and_flops(model, config.training.seq_len)
        self.loss_fn = spec.build_loss_fn(config.compile, parallel_dims=pd)

        gbs = config.training.global_batch_size
        if gbs < 0:
            gbs = config.training.local_batch_size * self.dp_degree
        assert gbs % (config.training.local_batch_size * self.dp_degree) == 0
        self.gradient_accumulation_steps = gbs // (config.training.local_batch_size * self.dp_degree)
        self.global_batch_size = gbs

        self.pp_has_first_stage = self.pp_has_last_stage = True
        self.pp_schedule = None
        if pd.pp_enabled:
            if spec.pipelining_fn is None:
                raise RuntimeError(f"Pipeline Parallel is enabled but {spec.name} does not support pipelining")
            (self.pp_schedule, self.model_parts, self.pp_has_first_stage, self.pp_has_last_stage) = spec.pipelining_fn(
                model, parallel_dims=pd, training=config.training, model_converters=config.model_converters,
                parallelism=config.parallelism, compile_config=config.compile, ac_config=config.activation_checkpoint,
                dump_folder=config.dump_folder, device=self.device, model_config=model_config,
                parallelize_fn=spec.parallelize_fn, loss_fn=self.loss_fn,
            )
        else:
            model = spec.parallelize_fn(
                model, parallel_dims=pd, training=config.training, model_converters=config.model_converters,
                parallelism=config.parallelism, compile_config=config.compile, ac_config=config.activation_checkpoint,
                dump_folder=config.dump_folder,
            )
            self.model_parts = [model]
        for m in self.model_parts:
            self._materialize(m)

        self.optimizers = config.optimizer.build(model_parts=self.model_parts)
        if spec.post_optimizer_build_fn is not None:
            spec.post_optimizer_build_fn(self.optimizers, self.model_parts, pd)
        self.lr_schedulers = config.lr_scheduler.build(optimizers=self.optimizers, training_steps=config.training.steps)
        self.optimizers.register_step_post_hook(lambda *a, **k: converters.post_optimizer_hook(self.model_parts))
        self.step = 0
        self.checkpointer = config.checkpoint.build(
            dataloader=None, model_parts=self.model_parts, optimizers=self.optimizers, lr_schedulers=self.lr_schedulers,
            states={"train_state": self},
            sd_adapter=(spec.state_dict_adapter(model_config, config.hf_assets_path) if spec.state_dict_adapter else None),
            base_folder=config.dump_folder,
        )
        loss_parallel = pd.tp_enabled and not config.parallelism.disable_loss_parallel
        self.train_context = dist_utils.get_train_context(loss_parallel)
        self.maybe_enable_amp = dist_utils.maybe_enable_amp(pd, config.training.mixed_precision_param, dev_type)
        logger.info(f"ForgeEngine ready: {spec.name} {spec.flavor}, {self.model_param_count:,} parameters")

    def _materialize(self, model) -> None:
        from torchtitan_b200.parallel import fsdp

        model.to_empty(device=self.device)
        with torch.no_grad():
            model.init_weights(buffer_device=None)
        model.train()
        fsdp.materialize(model)
        if self.parallel_dims.tp_enabled or self.parallel_dims.ep_enabled:
            from torchtitan_b200.parallel.tp import finalize_tp

            finalize_tp(model)

    def state_dict(self) -> dict[str, Any]:
        return {"step": self.step}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.step = state_dict["step"]

    def close(self) -> None:
        if getattr(self, "checkpointer", None):
            self.checkpointer.close()
