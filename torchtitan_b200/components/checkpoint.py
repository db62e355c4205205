"""Checkpoint manager on top of ``torch.distributed.checkpoint`` (DCP).

On-disk contract (identical to torchtitan/components/checkpoint.py so either framework loads the
other's checkpoints): directory ``<dump>/<folder>/step-<N>``; the model's parameters and
persistent buffers are *flattened at the top level* under their FQNs (:899-910); the other keys
are ``optimizer`` (flattened optimizer state), ``lr_scheduler``, ``dataloader`` and
``train_state`` (:52-56). A folder counts as a checkpoint when it contains ``.metadata`` (DCP) or
``model.safetensors.index.json`` (HF) (:832-861). Step-0 checkpoints hold the model only (seed
checkpoints, :798). Behaviours reproduced: interval / first-step / last-step rules (:975-988),
model-only last save with ``export_dtype`` and optional HF safetensors export (:943-973), async
modes ``async`` (background DCP save over a gloo group) and ``async_with_pinned_mem`` (stage to
pinned memory, then save from a worker; the trainer only waits for staging, :510-598, :821-830),
``keep_latest_k`` purge thread (:99-122, :1006-1029), ``initial_load_path`` /
``initial_load_model_only`` / ``initial_load_in_hf`` / ``exclude_from_loading`` / ``load_step`` /
``load_only`` (:719-819), and the fault-tolerance hooks: per-replica dataloader checkpoints and
live state transfer functions (:391-414, :870-897).
"""

from __future__ import annotations

import enum
import functools
import os
import queue
import re
import shutil
import threading
import time
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Any, Literal

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
import torch.nn as nn
from torch.distributed.checkpoint.stateful import Stateful

from torchtitan_b200.config import TORCH_DTYPE_MAP
from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.tools.logging import logger
from torchtitan_b200.tools.utils import GarbageCollection

MODEL = "model"
OPTIMIZER = "optimizer"
LR_SCHEDULER = "lr_scheduler"
DATALOADER = "dataloader"
TRAIN_STATE = "train_state"


class AsyncMode(str, enum.Enum):
    DISABLED = "disabled"
    ASYNC = "async"
    ASYNC_WITH_PINNED_MEM = "async_with_pinned_mem"


class ModelWrapper(Stateful):
    """All model parts presented as one flat ``{fqn: tensor}`` mapping (persistent state only)."""

    def __init__(self, model: nn.Module | list[nn.Module]) -> None:
        self.model = [model] if isinstance(model, nn.Module) else model
        self.cache_state_dict = self._get_state_dict()

    def _get_state_dict(self) -> dict[str, Any]:
        """Tensor- and expert-parallel shards appear with their full logical shape (``parallel/global_view.py``): the
        checkpoint does not depend on the layout that wrote it."""
        from torchtitan_b200.parallel.global_view import global_view, is_outer_sharded

        out: dict[str, Any] = {}
        for part in self.model:
            sd = part.state_dict()
            for name, p in part.named_parameters(remove_duplicate=False):
                if name in sd and is_outer_sharded(p):
                    sd[name] = global_view(p)
            out.update(sd)
        return out

    def state_dict(self) -> dict[str, Any]:
        return self.cache_state_dict

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        from torchtitan_b200.parallel.fsdp import fsdp_units
        from torchtitan_b200.parallel.global_view import is_outer_sharded, local_of

        for part in self.model:
            own = part.state_dict()
            sub = {k: v for k, v in state_dict.items() if k in own}
            with torch.no_grad():
                for name, p in part.named_parameters(remove_duplicate=False):
                    if name in sub and is_outer_sharded(p):
                        # a full-shape view: its local piece has this rank's layout (a distributed-checkpoint load has
                        # usually written it in place already, then this copy is a no-op)
                        src, dst = local_of(sub.pop(name)), local_of(p)
                        if tuple(src.shape) != tuple(dst.shape):
                            raise ValueError(f"{name}: cannot load a tensor of local shape {tuple(src.shape)} into a "
                                             f"shard of shape {tuple(dst.shape)}")
                        if src.data_ptr() != dst.data_ptr():
                            dst.copy_(src)
            part.load_state_dict(sub, strict=False)
            for u in fsdp_units(part):
                u.mark_params_updated()
        # parameters were copied in place, but buffers may have been re-bound: refresh the cache
        self.cache_state_dict = self._get_state_dict()


def _purge_worker(q: queue.Queue):
    """Deletes checkpoint folders handed over the queue until it receives ``None``."""
    while True:
        path = q.get()
        if path is None:
            return
        t0 = time.monotonic()
        logger.info(f"Checkpointer is deleting {path}.")
        shutil.rmtree(path, ignore_errors=True)
        logger.info("Checkpointer deleted %s in %.2f seconds.", path, time.monotonic() - t0)


class CheckpointManager(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        enable: bool = False
        enable_ft_dataloader_checkpoints: bool = True
        folder: str = "checkpoint"
        interval: int = 500
        initial_load_path: str | None = None
        """Checkpoint to start from when ``folder`` has none yet (model only unless overridden)."""
        initial_load_model_only: bool = True
        initial_load_in_hf: bool = False
        initial_load_in_hf_quantized: bool = False
        last_save_model_only: bool = True
        last_save_in_hf: bool = False
        export_dtype: Literal["float16", "bfloat16", "float32"] = "float32"
        async_mode: Literal["disabled", "async", "async_with_pinned_mem"] = "disabled"
        keep_latest_k: int = 10
        load_step: int = -1
        exclude_from_loading: list[str] = field(default_factory=list)
        enable_first_step_checkpoint: bool = False
        create_seed_checkpoint: bool = False
        load_only: bool = False

    def __init__(self, config: Config, *, dataloader, model_parts: list[nn.Module], optimizers, lr_schedulers,
                 states: dict[str, Any], sd_adapter=None, base_folder: str = "", ft_manager=None) -> None:
        self.enable = config.enable
        self.load_only = config.load_only
        self.states = states
        self.states.update({
            MODEL: ModelWrapper(model_parts),
            OPTIMIZER: optimizers,
            DATALOADER: dataloader,
            LR_SCHEDULER: lr_schedulers,
        })
        self.ft_manager = ft_manager.manager if ft_manager is not None and ft_manager.enabled else None
        self.enable_ft_dataloader_checkpoints = bool(self.ft_manager and config.enable_ft_dataloader_checkpoints)
        if self.ft_manager and not self.enable_ft_dataloader_checkpoints:
            logger.warning(
                "Fault tolerance is enabled but enable_ft_dataloader_checkpoints is False. "
                "Replicas may retrain over the same data multiple times."
            )
        if self.ft_manager:
            optimizers.init_cache_state_dict()
            live = (MODEL, OPTIMIZER, LR_SCHEDULER, TRAIN_STATE)
            self.ft_manager.set_state_dict_fns(
                lambda sd: [self.states[k].load_state_dict(v) for k, v in sd.items()],
                lambda: {k: v.state_dict() for k, v in self.states.items() if k in live},
            )
            self.ft_replica_id = ft_manager.replica_id
        mode = AsyncMode(config.async_mode.lower())
        self.enable_staging = (self.enable and mode == AsyncMode.ASYNC_WITH_PINNED_MEM) or self.enable_ft_dataloader_checkpoints
        if not self.enable and not self.enable_ft_dataloader_checkpoints:
            return
        self.ft_states = {DATALOADER: dataloader}
        self.async_mode = mode
        self.staging = False
        self.stager = None
        self.staging_future: Future | None = None
        self.save_future: Future | None = None
        self.folder = os.path.join(base_folder, config.folder)
        self.initial_load_model_only = config.initial_load_model_only
        self.initial_load_in_hf = config.initial_load_in_hf
        self.initial_load_in_hf_quantized = config.initial_load_in_hf_quantized
        self.initial_load_path = config.initial_load_path
        self.last_save_model_only = config.last_save_model_only
        self.last_save_in_hf = config.last_save_in_hf
        if self.last_save_in_hf:
            assert sd_adapter is not None, "checkpoint.last_save_in_hf is True, but sd_adapter is not provided."
        self.sd_adapter = sd_adapter
        self.export_dtype = TORCH_DTYPE_MAP[config.export_dtype]
        self.exclude_from_loading = config.exclude_from_loading
        self.interval = config.interval
        self.enable_first_step_checkpoint = config.enable_first_step_checkpoint
        self.load_step = config.load_step
        self.pg = None
        if mode != AsyncMode.DISABLED or self.enable_ft_dataloader_checkpoints:
            self.pg = dist.new_group(backend="gloo")
        self.keep_latest_k = config.keep_latest_k
        self.purge_thread = None
        if self.keep_latest_k > 0:
            if self.keep_latest_k == 1:
                raise ValueError(
                    "We need to maintain at least 2 checkpoint replicas, as the last one may be in the process of being saved."
                )
            self.purge_queue: queue.Queue = queue.Queue()
            self.purge_thread = threading.Thread(target=_purge_worker, args=(self.purge_queue,), daemon=True)
            self.purge_thread.start()
        logger.info(f"Checkpointing active. Checkpoints will be loaded from and saved to {self.folder}")

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def close(self):
        if getattr(self, "enable", False):
            t = getattr(self, "purge_thread", None)
            if t is not None and t.is_alive():
                self.purge_queue.put(None)
                t.join()
                self.purge_thread = None
            if getattr(self, "stager", None) is not None:
                self.stager.close()
                self.stager = None

    # ------------------------------------------------------------------ DCP calls
    def dcp_save(self, state_dict: dict[str, Any], checkpoint_id: str, async_mode: AsyncMode,
                 enable_garbage_collection: bool = False, to_hf: bool = False):
        """Save ``state_dict`` to ``checkpoint_id``; returns a future (or an ``AsyncSaveResponse``)
        for the async modes."""
        ret = None
        storage_writer = None
        if to_hf:
            assert self.sd_adapter is not None, "trying to save checkpoint in HF safetensors format, but sd_adapter is not provided."
            from torch.distributed.checkpoint import HuggingFaceStorageWriter

            state_dict = self.sd_adapter.to_hf(state_dict)
            mapping = self.sd_adapter.fqn_to_index_mapping
            if mapping:
                storage_writer = HuggingFaceStorageWriter(
                    path=os.path.join(checkpoint_id, "sharded"), save_distributed=True,
                    fqn_to_index_mapping=mapping, enable_consolidation=False,
                )
            else:
                storage_writer = HuggingFaceStorageWriter(path=checkpoint_id, save_distributed=True, enable_consolidation=True)
        kw = dict(storage_writer=storage_writer) if storage_writer is not None else {}
        cid = None if storage_writer is not None else checkpoint_id
        if async_mode == AsyncMode.ASYNC:
            ret = dcp.async_save(state_dict, checkpoint_id=cid, process_group=self.pg, **kw)
        elif async_mode == AsyncMode.ASYNC_WITH_PINNED_MEM:
            from torch.distributed.checkpoint.staging import DefaultStager, StagingOptions
            from torch.distributed.checkpoint.state_dict_saver import AsyncCheckpointerType

            if self.stager is None:
                self.stager = DefaultStager(StagingOptions(True, True, True, True))
            ret = dcp.async_save(
                state_dict, checkpoint_id=cid, process_group=self.pg,
                async_checkpointer_type=AsyncCheckpointerType.PROCESS, async_stager=self.stager, **kw,
            )
        else:
            ret = dcp.save(state_dict, checkpoint_id=cid, **kw)
        if to_hf and self.sd_adapter.fqn_to_index_mapping:
            from torch.distributed.checkpoint._consolidate_hf_safetensors import consolidate_safetensors_files_on_every_rank

            consolidate_safetensors_files_on_every_rank(
                input_dir=os.path.join(checkpoint_id, "sharded"), output_dir=checkpoint_id,
                fqn_to_index_mapping=self.sd_adapter.fqn_to_index_mapping, num_threads=5,
            )
        if enable_garbage_collection:
            GarbageCollection.collect("GC collection invoked by checkpointer.")
        return ret

    def dcp_load(self, state_dict: dict[str, Any], checkpoint_id: str, from_hf: bool, from_quantized: bool = False) -> None:
        if from_hf:
            assert self.sd_adapter is not None, "trying to load checkpoint in HF safetensors format, but sd_adapter is not provided."
            hf_sd = self.sd_adapter.to_hf(state_dict)
            dcp.load(hf_sd, storage_reader=self.sd_adapter.get_hf_storage_reader(checkpoint_id, from_quantized))
            state_dict = self.sd_adapter.from_hf(hf_sd)
            self.states[MODEL].load_state_dict(state_dict)
            return
        # DCP loads tensors in place and calls load_state_dict() on the Stateful entries itself;
        # the model's entries are flattened at the top level, so the model is told by hand.
        dcp.load(state_dict, checkpoint_id=checkpoint_id)
        if MODEL in self.states:
            model_sd = {k: v for k, v in state_dict.items() if k not in self.states}
            if model_sd:
                self.states[MODEL].load_state_dict(model_sd)

    # ------------------------------------------------------------------ save
    @torch.no_grad()
    def save(self, curr_step: int, last_step: bool = False) -> None:
        if self.enable_ft_dataloader_checkpoints:
            self._ft_save(curr_step)
        if not self._should_save(curr_step, last_step):
            return
        t0 = time.monotonic()
        if not self.ft_manager or self.ft_manager.participating_rank() == 0:
            logger.info("Saving the checkpoint (or staging if async is enabled).")
            checkpoint_id = self._create_checkpoint_id(curr_step)
            self._async_wait()
            if last_step:
                self._save_last_step(curr_step)
                return
            states = self._flattened_model_states_sd()
            if self.async_mode == AsyncMode.ASYNC_WITH_PINNED_MEM:
                GarbageCollection.collect("GC collection invoked by checkpointer.")
                result = self.dcp_save(states, checkpoint_id, self.async_mode)
                self.save_future = result.upload_completion
                self.staging_future = result.staging_completion
                self.staging = True
            elif self.async_mode == AsyncMode.ASYNC:
                GarbageCollection.collect("GC collection invoked by checkpointer.")
                self.save_future = self.dcp_save(states, checkpoint_id, self.async_mode)
                GarbageCollection.collect("GC collection invoked by checkpointer.")
            else:
                self.dcp_save(states, checkpoint_id, AsyncMode.DISABLED, enable_garbage_collection=True)
            self._purge_stale_checkpoints()
            logger.info("Finished saving the checkpoint (or staging if async is enabled) in %.2f seconds.", time.monotonic() - t0)
        elif self.ft_manager:
            logger.info("Replica %d doesn't save checkpoint.", self.ft_manager.participating_rank())

    def _save_last_step(self, curr_step: int) -> None:
        if self.last_save_model_only:
            states = dict(self.states[MODEL].state_dict())
            if self.export_dtype != torch.float32:
                states = {k: v.to(self.export_dtype) for k, v in states.items()}
            logger.info(f"Saving a model only checkpoint in {self.export_dtype} at last step, step {curr_step}.")
        else:
            logger.info(f"Saving a full checkpoint at last step, step {curr_step}.")
            states = self._flattened_model_states_sd()
        if self.last_save_in_hf:
            assert self.last_save_model_only, "Only model can be saved when saving in HF safetensors format."
        self.dcp_save(states, self._create_checkpoint_id(curr_step), AsyncMode.DISABLED,
                      enable_garbage_collection=True, to_hf=self.last_save_in_hf)

    def _flattened_model_states_sd(self, state_dict: dict[str, Any] | None = None) -> dict[str, Any]:
        src = state_dict if state_dict is not None else self.states
        out = {k: v for k, v in src.items() if k != MODEL}
        if MODEL in src:
            out.update(src[MODEL].state_dict())
        return out

    def will_save(self, curr_step: int, last_step: bool = False) -> bool:
        """Whether :meth:`save` would write a checkpoint for this step (the trainer checks the kernels' error words first)."""
        return self._should_save(curr_step, last_step)

    def _should_save(self, curr_step: int, last_step: bool = False) -> bool:
        if not self.enable or self.load_only:
            return False
        if curr_step == 1 and self.enable_first_step_checkpoint:
            return True
        return last_step or curr_step % self.interval == 0

    def _create_checkpoint_id(self, step: int, folder: str = "") -> str:
        return os.path.join(folder or self.folder, f"step-{step}")

    # ------------------------------------------------------------------ load
    @torch.no_grad()
    def load(self, step: int = -1) -> bool:
        if self.enable_ft_dataloader_checkpoints:
            self._ft_load()
        if not self.enable:
            return False
        if step == -1:
            step = self.load_step
        model_only = False
        from_hf = False
        from_quantized = False
        if not os.path.exists(self.folder):
            model_only = self.initial_load_model_only
            from_hf = self.initial_load_in_hf
            from_quantized = self.initial_load_in_hf_quantized
            if from_hf:
                assert model_only, "Only model can be loaded when loading from HF's safetensors checkpoint."
            if from_quantized:
                assert from_hf, "Quantized checkpoint can only be loaded from HuggingFace format."
            if self.initial_load_path:
                checkpoint_id = self.initial_load_path
                if not os.path.isdir(checkpoint_id):
                    raise ValueError(f"checkpoint.initial_load_path is specified but the path is not valid: {checkpoint_id}")
                if from_hf:
                    logger.info(f"loading from HF safetensors from --checkpoint.initial_load_path: {checkpoint_id}")
            elif from_hf:
                checkpoint_id = self.sd_adapter.hf_assets_path
                if not os.path.isdir(checkpoint_id):
                    raise ValueError(
                        f"model.hf_assets_path is being used to load HF weights but the path is not valid: {checkpoint_id}. "
                        "Either make sure hf_assets_path is correct or provide a valid checkpoint.initial_load_path"
                    )
                logger.info(f"loading HF safetensors from --model.hf_assets_path: {checkpoint_id}")
            else:
                return False
        else:
            if self.initial_load_path:
                logger.warning(
                    "checkpoint.initial_load_path is provided but the checkpoint.folder exists. "
                    f"Checkpointer will use the checkpoints from the checkpoint.folder {self.folder}."
                )
            if self.initial_load_in_hf:
                logger.warning(
                    "checkpoint.initial_load_in_hf is True but the checkpoint.folder exists. "
                    "Checkpointer will not load from HF safetensors"
                )
            step = self._find_load_step() if step == -1 else step
            if step == -1:
                return False
            model_only = step == 0
            checkpoint_id = self._create_checkpoint_id(step)
            if not os.path.isdir(checkpoint_id):
                raise FileNotFoundError(f"--checkpoint.load_step={step} but checkpoint {checkpoint_id} is not found.")
        logger.info(f"Loading the checkpoint from {checkpoint_id}.")
        t0 = time.monotonic()
        states = self._states_to_load(model_only)
        self.dcp_load(states, checkpoint_id=checkpoint_id, from_hf=from_hf, from_quantized=from_quantized)
        GarbageCollection.collect("GC collection for checkpoint loading.")
        logger.info(f"Finished loading the checkpoint in {time.monotonic() - t0:.2f} seconds.")
        return True

    def _states_to_load(self, model_only: bool) -> dict[str, Any]:
        if model_only:
            return dict(self.states[MODEL].state_dict())
        for k in self.exclude_from_loading:
            if k not in self.states:
                raise ValueError(f"{k} not found in state_dict.")
        keep = {k: v for k, v in self.states.items() if k not in self.exclude_from_loading}
        out = self._flattened_model_states_sd(keep)
        if self.ft_manager:
            out.pop(DATALOADER, None)
        return out

    def _find_load_step(self, folder: str = "") -> int:
        folder = folder or self.folder
        if not os.path.isdir(folder):
            return -1
        steps = []
        for name in os.listdir(folder):
            m = re.fullmatch(r"step-(\d+)", name)
            if not m:
                continue
            path = os.path.join(folder, name)
            if os.path.isfile(os.path.join(path, ".metadata")) or os.path.isfile(os.path.join(path, "model.safetensors.index.json")):
                steps.append(int(m.group(1)))
        return max(steps) if steps else -1

    # ------------------------------------------------------------------ async helpers
    def maybe_wait_for_staging(self) -> None:
        """Block until the pinned-memory copy of the last async save is complete (the optimizer is
        about to overwrite the parameters)."""
        if getattr(self, "enable_staging", False) and getattr(self, "staging", False):
            if self.staging_future is not None:
                self.staging_future.result()
            self.staging = False

    def _async_wait(self) -> None:
        if self.async_mode in (AsyncMode.ASYNC, AsyncMode.ASYNC_WITH_PINNED_MEM) and self.save_future is not None:
            self.save_future.result()
            self.save_future = None

    def _purge_stale_checkpoints(self) -> None:
        if not (self.keep_latest_k > 0 and dist.get_rank() == 0 and os.path.isdir(self.folder)):
            return
        if self.ft_manager and self.ft_manager.participating_rank() != 0:
            return
        found = []
        for name in os.listdir(self.folder):
            m = re.fullmatch(r"step-(\d+)", name)
            if m:
                found.append((int(m.group(1)), os.path.join(self.folder, name)))
        found.sort()
        for _, path in found[: -self.keep_latest_k]:
            assert self.purge_thread is not None
            self.purge_queue.put(path)

    # ------------------------------------------------------------------ fault tolerance
    def _ft_folder(self) -> str:
        return os.path.join(self.folder, f"ft-replicat-{self.ft_replica_id}")

    def _ft_save(self, step: int) -> None:
        begin = time.monotonic()
        self._async_wait()
        cid = self._create_checkpoint_id(step, folder=self._ft_folder())
        self.save_future = self.dcp_save(self.ft_states, cid, AsyncMode.ASYNC)
        logger.info(f"Staging ft checkpoint took {time.monotonic() - begin} secs.")

    def _ft_load(self) -> None:
        step = self._find_load_step(folder=self._ft_folder())
        if step == -1:
            return
        begin = time.monotonic()
        logger.info(f"Loading the FT checkpoint at step {step}.")
        cid = self._create_checkpoint_id(step, folder=self._ft_folder())
        dcp.load(self.ft_states, checkpoint_id=cid)
        GarbageCollection.collect("GC collection for checkpoint loading.")
        logger.info(f"Finished loading the ft checkpoint in {time.monotonic() - begin:.2f} seconds.")
