"""``Trainer``: builds every component of a job from a ``Trainer.Config`` and runs the loop.

Public surface and override points follow torchtitan/trainer.py:57-868: nested ``Config`` with
the sections ``profiling, metrics, tokenizer, dataloader, model_converters, optimizer,
lr_scheduler, training, parallelism, checkpoint, activation_checkpoint, compile, comm,
validator, debug``; methods ``batch_generator``, ``post_dataloading_process``,
``forward_backward_step``, ``train_step``, ``train``, ``state_dict/load_state_dict`` (``{step,
ntokens_seen}``) and ``close``. Construction order (:193-504): device and process group ->
ParallelDims -> determinism -> tokenizer, dataloader -> model on ``meta`` -> converters ->
metrics/FLOPs -> loss -> gradient accumulation -> pipeline split or ``parallelize_fn`` ->
``to_empty`` + ``init_weights`` -> optimizers (+ post-build hook) -> LR schedulers ->
checkpointer -> train context -> validator.

Numerics contract (:679-687): the loss is ``sum(CE) / global_valid_tokens`` where the
denominator counts labels != -100 over *all* data-parallel ranks and micro-batches of the step,
and FSDP does not divide gradients.

Differences that matter on B200: the token count stays a device scalar (no ``.item()`` per
step; the only host syncs are on logging steps), batches are copied from pinned memory with
non-blocking copies, and each step can be timed on the device with CUDA events (metric
``time_metrics/device_step(ms)``).
"""

from __future__ import annotations

import contextlib
import dataclasses
import json
import os
import time
from dataclasses import asdict, dataclass, field
from datetime import timedelta
from typing import Annotated, Any, Iterable, Iterator

import torch
import torch.distributed as dist
import tyro
from torch.distributed.checkpoint.stateful import Stateful
from torch.distributed.elastic.multiprocessing.errors import record

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.dataloader import BaseDataLoader, DataloaderExhaustedError
from torchtitan_b200.components.loss import IGNORE_INDEX
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor, ensure_pp_loss_visible
from torchtitan_b200.components.optimizer import OptimizersContainer, OptimizersInBackwardContainer
from torchtitan_b200.components.tokenizer import BaseTokenizer, HuggingFaceTokenizer
from torchtitan_b200.components.validate import Validator
from torchtitan_b200.config import (
    TORCH_DTYPE_MAP,
    ActivationCheckpointConfig,
    CommConfig,
    CompileConfig,
    Configurable,
    DebugConfig,
    ParallelismConfig,
    TrainingConfig,
)
from torchtitan_b200.parallel import ParallelDims
from torchtitan_b200.parallel import utils as dist_utils
from torchtitan_b200.protocols.model_converter import ModelConvertersContainer
from torchtitan_b200.protocols.model_spec import ModelSpec
from torchtitan_b200.tools import utils
from torchtitan_b200.tools.logging import logger
from torchtitan_b200.tools.profiling import ProfilingConfig, maybe_enable_memory_snapshot, maybe_enable_profiling


class Trainer(Stateful, Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        model_spec: Annotated[ModelSpec | None, tyro.conf.Suppress] = None
        """Set by the config registry function, never from the command line."""
        hf_assets_path: str = "./tests/assets/tokenizer"
        """Folder with tokenizer files (and optionally HF weights / index / config)."""
        dump_folder: str = "./outputs"
        profiling: ProfilingConfig = field(default_factory=ProfilingConfig)
        metrics: MetricsProcessor.Config = field(default_factory=MetricsProcessor.Config)
        tokenizer: BaseTokenizer.Config | None = field(default_factory=HuggingFaceTokenizer.Config)
        dataloader: BaseDataLoader.Config = field(default_factory=BaseDataLoader.Config)
        model_converters: ModelConvertersContainer.Config = field(default_factory=ModelConvertersContainer.Config)
        optimizer: OptimizersContainer.Config = field(default_factory=OptimizersContainer.Config)
        lr_scheduler: LRSchedulersContainer.Config = field(default_factory=LRSchedulersContainer.Config)
        training: TrainingConfig = field(default_factory=TrainingConfig)
        parallelism: ParallelismConfig = field(default_factory=ParallelismConfig)
        checkpoint: CheckpointManager.Config = field(default_factory=CheckpointManager.Config)
        activation_checkpoint: ActivationCheckpointConfig = field(default_factory=ActivationCheckpointConfig)
        compile: CompileConfig = field(default_factory=CompileConfig)
        comm: CommConfig = field(default_factory=CommConfig)
        validator: Validator.Config = field(default_factory=Validator.Config)
        debug: DebugConfig = field(default_factory=DebugConfig)

        def __post_init__(self):
            if isinstance(self.optimizer, OptimizersInBackwardContainer.Config):
                if self.parallelism.expert_parallel_degree > 1:
                    raise NotImplementedError("Optimizers in backward is not supported with Expert Parallel.")
                if self.parallelism.pipeline_parallel_degree > 1:
                    raise NotImplementedError("Optimizers in backward is not supported with Pipeline Parallel.")

        def to_dict(self) -> dict[str, Any]:
            d: dict[str, Any] = {}
            for f in dataclasses.fields(self):
                v = getattr(self, f.name)
                if f.name == "model_spec":
                    d[f.name] = None if v is None else {"name": v.name, "flavor": v.flavor}
                elif hasattr(v, "to_dict"):
                    d[f.name] = v.to_dict()
                elif dataclasses.is_dataclass(v):
                    d[f.name] = asdict(v)
                else:
                    d[f.name] = v
            return d

        def maybe_log(self) -> None:
            if self.debug.print_config:
                logger.info(f"Running with configs: {json.dumps(self.to_dict(), indent=2, ensure_ascii=False, default=str)}")
            if self.debug.save_config_file is not None:
                path = os.path.join(self.dump_folder, self.debug.save_config_file)
                if dist.is_initialized():
                    if dist.get_rank() == 0:
                        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
                        with open(path, "w") as f:
                            json.dump(self.to_dict(), f, indent=2, default=str)
                    logger.info(f"Saved job configs to {path}")
                else:
                    logger.warning("Job configs logging is disabled due to torch.distributed not initialized.")

    # ------------------------------------------------------------------ construction
    @record
    def __init__(self, config: Config):
        self.config = config
        assert config.model_spec is not None, "model_spec must be set before creating Trainer"
        spec = config.model_spec
        self.model_spec = spec
        logger.info(f"Starting job: {spec.name} {spec.flavor}")

        dev_type = utils.device_type
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.device = torch.device(f"{dev_type}:{local_rank}") if dev_type == "cuda" else torch.device("cpu")
        if dev_type == "cuda":
            torch.cuda.set_device(self.device)

        self.parallel_dims = pd = self.init_distributed()
        self._post_init_distributed()
        if pd.dp_enabled:
            self.dp_degree = pd.dim_size("batch")
            self.dp_rank = pd.coordinate("batch", dist.get_rank())
        else:
            self.dp_degree, self.dp_rank = 1, 0

        self.gc_handler = utils.GarbageCollection(gc_freq=config.training.gc_freq, debug=config.training.gc_debug)
        # locally sharded (TP / EP) parameters are plain tensors: ranks along those dimensions need their
        # own random streams; replicated parameters are broadcast afterwards (tp.finalize_tp)
        seed_dims = ["pp"] + (["tp"] if pd.tp_enabled else []) + (["ep"] if pd.ep_enabled else [])
        self.base_seed = dist_utils.set_determinism(pd, self.device, config.debug, distinct_seed_mesh_dims=seed_dims)
        config.maybe_log()

        # ---- data ---------------------------------------------------------------------
        self.tokenizer = (
            config.tokenizer.build(tokenizer_path=config.hf_assets_path) if config.tokenizer is not None else None
        )
        self.model_config = model_config = spec.model
        model_config.update_from_config(trainer_config=config)
        self.dataloader = self._build_dataloader(config.dataloader, config.training.local_batch_size)

        # ---- model on meta ----------------------------------------------------------------
        logger.info(f"Building {spec.name} {spec.flavor} with {model_config!r}")
        with torch.device("meta"), utils.set_default_dtype(TORCH_DTYPE_MAP[config.training.dtype]):
            model = model_config.build()
        converters = config.model_converters.build(parallel_dims=pd, model_compile_enabled=config.compile.enable)
        converters.convert(model)
        self.model_converters = converters

        self.metrics_processor = config.metrics.build(
            parallel_dims=pd, dump_folder=config.dump_folder,
            pp_schedule=config.parallelism.pipeline_parallel_schedule, config_dict=config.to_dict(),
            has_quantization=bool(config.model_converters.converters),
        )
        color = self.metrics_processor.color
        nparams, flops_per_token = model_config.get_nparams_and_flops(model, config.training.seq_len)
        self.metrics_processor.num_flops_per_token = flops_per_token
        logger.info(f"{color.blue}Model {spec.name} {spec.flavor} {color.red}size: {nparams:,} total parameters{color.reset}")

        self.loss_fn = spec.build_loss_fn(config.compile, parallel_dims=pd)

        # ---- batch arithmetic ---------------------------------------------------------------
        gbs = config.training.global_batch_size
        if gbs < 0:
            gbs = config.training.local_batch_size * self.dp_degree
        assert gbs > 0
        assert gbs % (config.training.local_batch_size * self.dp_degree) == 0, (
            f"global batch size must be multiple of local batch size times data-parallel degree "
            f"({gbs} % ({config.training.local_batch_size} * {self.dp_degree}) != 0)"
        )
        self.gradient_accumulation_steps = gbs // (config.training.local_batch_size * self.dp_degree)
        assert self.gradient_accumulation_steps > 0
        self.global_batch_size = gbs

        # ---- parallelise ----------------------------------------------------------------------
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
            del model
            for m in self.model_parts:
                self._materialize(m)
            ensure_pp_loss_visible(pd, config.parallelism.pipeline_parallel_schedule, color)
        else:
            from torchtitan_b200.ops.wgrad_store import WeightGradStore

            WeightGradStore.enabled = False      # a pipeline job built earlier in this process may have left it on
            model = spec.parallelize_fn(
                model, parallel_dims=pd, training=config.training, model_converters=config.model_converters,
                parallelism=config.parallelism, compile_config=config.compile, ac_config=config.activation_checkpoint,
                dump_folder=config.dump_folder,
            )
            self._materialize(model)
            self.model_parts = [model]
        self.metrics_processor.model_parts = self.model_parts

        mem = self.metrics_processor.device_memory_monitor.get_peak_stats()
        logger.info(f"{dev_type.upper()} memory usage for model: {mem.max_reserved_gib:.2f}GiB({mem.max_reserved_pct:.2f}%)")

        # ---- optimizer / schedule / checkpoint -----------------------------------------------------
        self.optimizers = self._build_optimizers()
        if spec.post_optimizer_build_fn is not None:
            spec.post_optimizer_build_fn(self.optimizers, self.model_parts, pd)
        self.lr_schedulers = config.lr_scheduler.build(optimizers=self.optimizers, training_steps=config.training.steps)
        self.optimizers.register_step_post_hook(lambda *a, **k: converters.post_optimizer_hook(self.model_parts))
        self.metrics_processor.optimizers = self.optimizers
        self.metrics_processor.lr_schedulers = self.lr_schedulers

        from torchtitan_b200.components.optimizer import ShardAdamW

        # the flat-shard optimizer can apply the clip coefficient itself (one pass less over the gradients)
        self._fold_clip = all(isinstance(o, ShardAdamW) and not o.has_loose_params for o in self.optimizers.optimizers)
        self.step = 0
        self.ntokens_seen = 0
        self.checkpointer = config.checkpoint.build(
            dataloader=self.dataloader, model_parts=self.model_parts, optimizers=self.optimizers,
            lr_schedulers=self.lr_schedulers, states={"train_state": self},
            sd_adapter=(spec.state_dict_adapter(model_config, config.hf_assets_path) if spec.state_dict_adapter else None),
            base_folder=config.dump_folder,
        )

        loss_parallel = pd.tp_enabled and not config.parallelism.disable_loss_parallel
        self.train_context = dist_utils.get_train_context(loss_parallel)
        self.maybe_enable_amp = dist_utils.maybe_enable_amp(pd, config.training.mixed_precision_param, dev_type)

        self.validator = None
        if config.validator.enable:
            self.validator = config.validator.build(
                parallelism=config.parallelism, dp_world_size=self.dp_degree, dp_rank=self.dp_rank,
                tokenizer=self.tokenizer, parallel_dims=pd, loss_fn=self.loss_fn,
                validation_context=self.train_context, maybe_enable_amp=self.maybe_enable_amp,
                metrics_processor=self.metrics_processor, seq_len=config.training.seq_len,
                local_batch_size=config.training.local_batch_size, pp_schedule=self.pp_schedule,
                pp_has_first_stage=self.pp_has_first_stage, pp_has_last_stage=self.pp_has_last_stage,
                model_vocab_size=getattr(model_config, "vocab_size", None),
            )
        logger.info(
            f"Trainer is initialized with local batch size {config.training.local_batch_size}, global batch size "
            f"{gbs}, gradient accumulation steps {self.gradient_accumulation_steps}, sequence length "
            f"{config.training.seq_len}, total steps {config.training.steps} (warmup {config.lr_scheduler.warmup_steps})"
        )

    # ---- extension points used by experiment trainers (fault tolerance, forge, flux) -------------
    def _post_init_distributed(self) -> None:
        """Runs right after the process groups exist and before anything else is built."""

    def _dataloader_dp_info(self) -> tuple[int, int]:
        """(degree, rank) by which the dataset is split; replica-group trainers widen it."""
        return self.dp_degree, self.dp_rank

    def _build_optimizers(self):
        return self.config.optimizer.build(model_parts=self.model_parts)

    def _build_dataloader(self, dl_config, local_batch_size: int):
        dp_degree, dp_rank = self._dataloader_dp_info()
        return dl_config.build(
            dp_world_size=dp_degree, dp_rank=dp_rank, tokenizer=self.tokenizer,
            seq_len=self.config.training.seq_len, local_batch_size=local_batch_size,
            model_vocab_size=getattr(self.model_config, "vocab_size", None),
        )

    def _materialize(self, model: torch.nn.Module) -> None:
        from torchtitan_b200.parallel import fsdp

        init_device = "cpu" if self.config.training.enable_cpu_offload else self.device
        model.to_empty(device=init_device)
        with torch.no_grad():
            model.init_weights(buffer_device=self.device if self.config.training.enable_cpu_offload else None)
        model.train()
        fsdp.materialize(model)
        if self.parallel_dims.tp_enabled or self.parallel_dims.ep_enabled:
            from torchtitan_b200.parallel.tp import finalize_tp

            finalize_tp(model)

    def init_distributed(self) -> ParallelDims:
        c = self.config
        world = dist_utils.init_distributed(
            c.comm, enable_cpu_backend=c.training.enable_cpu_offload, base_folder=c.dump_folder,
        )
        p = c.parallelism
        return ParallelDims(
            dp_shard=p.data_parallel_shard_degree, dp_replicate=p.data_parallel_replicate_degree,
            cp=p.context_parallel_degree, tp=p.tensor_parallel_degree, pp=p.pipeline_parallel_degree,
            ep=p.expert_parallel_degree, etp=p.expert_tensor_parallel_degree, world_size=world,
        )

    # ------------------------------------------------------------------ data
    def batch_generator(self, data_iterable: Iterable) -> Iterator[tuple[dict[str, torch.Tensor], torch.Tensor]]:
        it = iter(data_iterable)
        while True:
            t0 = time.perf_counter()
            try:
                batch = next(it)
            except StopIteration as ex:
                raise DataloaderExhaustedError() from ex
            input_dict, labels = batch
            self.ntokens_seen += labels.numel()
            self.metrics_processor.ntokens_since_last_log += labels.numel()
            self.metrics_processor.data_loading_times.append(time.perf_counter() - t0)
            yield input_dict, labels

    def post_dataloading_process(self, input_dict: dict[str, torch.Tensor], labels: torch.Tensor):
        """Split a batch into (inputs, labels, extra_inputs, extra_kwargs). ``extra_kwargs``
        (attention masks, positions) go to every pipeline stage; ``extra_inputs`` only to the first."""
        return prepare_batch(
            input_dict, labels, self.model_parts, self.tokenizer, self.parallel_dims, self.config.parallelism
        )

    # ------------------------------------------------------------------ step
    def forward_backward_step(self, *, input_dict: dict[str, torch.Tensor], labels: torch.Tensor,
                              global_valid_tokens: torch.Tensor) -> torch.Tensor:
        inputs, labels, extra_inputs, extra_kwargs = self.post_dataloading_process(input_dict, labels)
        if self.parallel_dims.pp_enabled:
            # each micro-batch loss is multiplied by 1 / global_valid_tokens before its backward
            scale = 1.0 / global_valid_tokens
            with self.train_context():
                targets, losses = (labels, []) if self.pp_has_last_stage else (None, None)
                if self.pp_has_first_stage:
                    self.pp_schedule.step(inputs, **extra_inputs, **extra_kwargs, target=targets, losses=losses,
                                          loss_scale=scale)
                else:
                    self.pp_schedule.step(**extra_kwargs, target=targets, losses=losses, loss_scale=scale)
            if self.pp_has_last_stage:
                loss = torch.sum(torch.stack(losses)).to(self.device)
            else:
                loss = torch.tensor([-1.0], device=self.device)
            return loss
        with self.train_context():
            assert len(self.model_parts) == 1
            with self.maybe_enable_amp:
                pred = self.model_parts[0](inputs, **extra_inputs, **extra_kwargs)
                loss_sum = self.loss_fn(pred, labels)
            loss = loss_sum / global_valid_tokens
            del pred
            loss.backward()
        return loss

    def train_step(self, data_iterator) -> None:
        self.optimizers.zero_grad()
        pd = self.parallel_dims
        lr = self.lr_schedulers.schedulers[0].get_last_lr()[0]

        microbatches = []
        host_valid, dev_valid = 0, None
        for _ in range(self.gradient_accumulation_steps):
            input_dict, labels = next(data_iterator)
            n = (labels != IGNORE_INDEX).sum()
            if labels.device.type == "cpu":
                host_valid += int(n)           # host tensor: counting it is not a device synchronisation
            else:
                dev_valid = n if dev_valid is None else dev_valid + n
            microbatches.append((input_dict, labels))
        # the denominator is built and stays on the device: no device -> host read anywhere in the step
        local_valid = torch.tensor(float(host_valid), dtype=torch.float32, device=self.device)
        if dev_valid is not None:
            local_valid = local_valid + dev_valid.to(torch.float32)
        global_valid_tokens = local_valid.clone()
        if pd.dp_enabled:
            dist.all_reduce(global_valid_tokens, group=pd.get_mesh("batch").get_group())

        accumulated = []
        for input_dict, labels in microbatches:
            input_dict = {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in input_dict.items()}
            labels = labels.to(self.device, non_blocking=True)
            loss = self.forward_backward_step(input_dict=input_dict, labels=labels, global_valid_tokens=global_valid_tokens)
            accumulated.append(loss.detach())

        grad_norm = dist_utils.clip_grad_norm_(
            [p for m in self.model_parts for p in m.parameters()], self.config.training.max_norm,
            foreach=True, pp_mesh=pd.get_optional_mesh("pp"), ep_enabled=pd.ep_enabled,
            fold_into_optimizer=self._fold_clip,
        )
        self.checkpointer.maybe_wait_for_staging()
        self.optimizers.step()
        self.lr_schedulers.step()
        self.last_loss = torch.sum(torch.stack(accumulated))
        self.last_grad_norm = grad_norm

        if not self.metrics_processor.should_log(self.step):
            return
        loss = self.last_loss
        if pd.dp_cp_enabled:
            loss = loss.detach()
            loss_mesh = pd.get_optional_mesh("loss")
            # this rank's loss sum over the valid tokens of its own batch, as in the reference
            # (torchtitan/trainer.py:764-768)
            local_avg = loss * global_valid_tokens / torch.clamp(local_valid, min=1.0)
            global_avg_loss = dist_utils.dist_sum(loss, loss_mesh)
            global_max_loss = dist_utils.dist_max(local_avg, loss_mesh)
            global_ntokens = dist_utils.dist_sum(
                torch.tensor(self.ntokens_seen, dtype=torch.int64, device=self.device), loss_mesh
            )
        else:
            global_avg_loss = global_max_loss = loss.detach().item()
            global_ntokens = self.ntokens_seen
        extra = {"n_tokens_seen": global_ntokens, "lr": lr}
        self.metrics_processor.log(self.step, global_avg_loss, global_max_loss, float(grad_norm), extra_metrics=extra)
        self._raise_on_kernel_errors()

    def _kernel_error_words(self, sync: bool = False) -> dict:
        """Error words of the native kernel families that are set ({} on CPU or without the native library)."""
        if self.device.type != "cuda":
            return {}
        from torchtitan_b200.ops import native

        if not native.available():
            return {}
        if sync:
            torch.cuda.synchronize()
        return native.kernel_errors()

    def _raise_on_kernel_errors(self, sync: bool = False) -> None:
        """The CUDA kernels of this framework bound every wait (peer flags, mbarriers, arrival counters); one that gives
        up sets a bit in its family's error word and returns, so the step finishes with wrong numbers instead of
        hanging. The words are read at log steps (the host has just synchronised for the loss) and, with ``sync``,
        before every checkpoint save and validation pass, so that no checkpoint is written from such a step."""
        errs = self._kernel_error_words(sync)
        ep = errs.get("ep")
        if ep and ep[0] == 2:
            # not an expired wait: the fixed-capacity expert exchange (hybridep_non_blocking_expert_capacity_factor) met
            # more rows than its receive buffer holds and dropped the rest, which is that mode's contract
            logger.warning(f"step {self.step}: the expert exchange dropped tokens since the last log: rank {ep[1]} was sent "
                           f"{ep[3]} rows, its receive buffer holds {ep[2]}; raise the capacity factor or use the lossless default")
            errs = {k: v for k, v in errs.items() if k != "ep"}
        if errs:
            raise RuntimeError(f"step {self.step}: a kernel gave up on a bounded wait (family -> error word): {errs}. "
                               "The results of the steps since the last log are not trustworthy.")

    # ------------------------------------------------------------------ loop
    @record
    def train(self):
        config = self.config
        self.checkpointer.load(step=config.checkpoint.load_step)
        logger.info(f"Training starts at step {self.step + 1}")
        leaf = ""
        data_iterator = self.batch_generator(self.dataloader)
        with maybe_enable_profiling(config.profiling, global_step=self.step, base_folder=config.dump_folder, leaf_folder=leaf) as prof, \
                maybe_enable_memory_snapshot(config.profiling, global_step=self.step, base_folder=config.dump_folder) as memprof:
            while self.should_continue_training():
                self.step += 1
                self.gc_handler.run(self.step)
                ev = None
                if self.device.type == "cuda":
                    ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    ev[0].record()
                try:
                    self.train_step(data_iterator)
                except DataloaderExhaustedError:
                    logger.warning("Ran out of data; last step was canceled.")
                    break
                if ev is not None:
                    ev[1].record()
                    self._pending_step_events = getattr(self, "_pending_step_events", []) + [ev]
                    self._drain_step_events()
                last = self.step == config.training.steps
                will_validate = self.validator is not None and self.validator.should_validate(self.step)
                if will_validate or self.checkpointer.will_save(self.step, last_step=last):
                    # a kernel that gave up on a bounded wait leaves wrong numbers behind: never persist or score them
                    self._raise_on_kernel_errors(sync=True)
                self.checkpointer.save(self.step, last_step=last)
                if will_validate:
                    self.validator.validate(self.model_parts, self.step)
                if prof is not None:
                    prof.step()
                if memprof is not None:
                    memprof.step()
                if self.step == 1:
                    dist_utils.set_pg_timeouts(timedelta(seconds=config.comm.train_timeout_seconds), self.parallel_dims)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        if dist.get_rank() == 0:
            logger.info("Sleeping 2 seconds for other ranks to complete")
            time.sleep(2)
        logger.info("Training completed")

    def _drain_step_events(self):
        keep = []
        for a, b in self._pending_step_events:
            if b.query():
                self.metrics_processor.device_step_ms.append(a.elapsed_time(b))
            else:
                keep.append((a, b))
        self._pending_step_events = keep[-8:]

    def should_continue_training(self) -> bool:
        return self.step < self.config.training.steps

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict[str, Any]:
        return {"step": self.step, "ntokens_seen": self.ntokens_seen}

    def load_state_dict(self, state_dict: dict[str, Any]):
        self.step = state_dict["step"]
        self.ntokens_seen = state_dict["ntokens_seen"]

    def close(self) -> None:
        if getattr(self, "checkpointer", None):
            self.checkpointer.close()
        if getattr(self, "metrics_processor", None):
            self.metrics_processor.close()


def prepare_batch(input_dict, labels, model_parts, tokenizer, parallel_dims, parallelism):
    """Shared by Trainer and Validator: masks, positions and context-parallel sharding."""
    inputs = input_dict["input"]
    extra_inputs = {k: v for k, v in input_dict.items() if k != "input"}
    extra_kwargs: dict[str, Any] = {}
    get_masks = getattr(model_parts[0], "get_attention_masks", None)
    if get_masks is not None:
        try:
            extra_kwargs["attention_masks"] = get_masks(input_batch=inputs, tokenizer=tokenizer, extra_inputs=extra_inputs)
        except TypeError:
            pass
    if parallel_dims.cp_enabled:
        from torchtitan_b200.parallel.cp import prepare_context_parallel_input

        inputs, labels, extra_kwargs = prepare_context_parallel_input(
            inputs, labels, extra_kwargs, parallel_dims.get_mesh("cp"), inputs.device,
            parallelism.context_parallel_load_balancer,
        )
    return inputs, labels, extra_inputs, extra_kwargs
