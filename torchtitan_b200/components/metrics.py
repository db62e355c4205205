"""Training metrics: throughput, MFU, memory, loss; console + TensorBoard / W&B sinks.

Parity: torchtitan/components/metrics.py:39-582. Formulae: ``tps = tokens_since_last_log /
(dt * cp * tp * pp)`` (per device), ``tflops = flops_per_token * tps / 1e12``, ``mfu = 100 *
flops_per_token * tps / peak`` (omitted when quantised converters are active); metric names
``loss_metrics/global_avg_loss``, ``loss_metrics/global_max_loss``, ``grad_norm``,
``throughput(tps)``, ``tflops``, ``mfu(%)``, ``time_metrics/*``, ``memory/*``; log on step 1 and
every ``log_freq`` steps; with pipeline parallel the logging rank is the first rank of the last
stage (the only stage that has the loss). Additions: per-layer MoE token histograms
(``moe/layer_<i>/tokens_per_expert``) and a device-timed step time.
"""

from __future__ import annotations

import os
import time
from collections import namedtuple
from dataclasses import dataclass
from datetime import datetime
from typing import Any

import torch

from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.tools import utils
from torchtitan_b200.tools.logging import logger

DeviceMemStats = namedtuple(
    "DeviceMemStats",
    ["max_active_gib", "max_active_pct", "max_reserved_gib", "max_reserved_pct", "num_alloc_retries", "num_ooms"],
)


class DeviceMemoryMonitor:
    def __init__(self, device: str | None = None):
        self.on_gpu = torch.cuda.is_available()
        if self.on_gpu:
            self.device = torch.device(device or f"cuda:{torch.cuda.current_device()}")
            self.device_name = torch.cuda.get_device_name(self.device)
            self.device_index = torch.cuda.current_device()
            self.device_capacity = torch.cuda.get_device_properties(self.device).total_memory
        else:
            import psutil

            self.device = torch.device("cpu")
            self.device_name = "cpu"
            self.device_index = 0
            self.device_capacity = psutil.virtual_memory().total
        self.device_capacity_gib = self._to_gib(self.device_capacity)
        self.reset_peak_stats()

    @staticmethod
    def _to_gib(b):
        return b / (1024**3)

    def _to_pct(self, b):
        return 100 * b / self.device_capacity

    def get_peak_stats(self) -> DeviceMemStats:
        if not self.on_gpu:
            import psutil

            rss = psutil.Process().memory_info().rss
            return DeviceMemStats(self._to_gib(rss), self._to_pct(rss), self._to_gib(rss), self._to_pct(rss), 0, 0)
        info = torch.cuda.memory_stats(self.device)
        act, res = info.get("active_bytes.all.peak", -1), info.get("reserved_bytes.all.peak", -1)
        retries, ooms = info.get("num_alloc_retries", -1), info.get("num_ooms", -1)
        if retries > 0:
            logger.warning(f"{retries} {self.device_name} memory allocation retries.")
        if ooms > 0:
            logger.warning(f"{ooms} {self.device_name} OOM errors thrown.")
        return DeviceMemStats(self._to_gib(act), self._to_pct(act), self._to_gib(res), self._to_pct(res), retries, ooms)

    def reset_peak_stats(self):
        if self.on_gpu:
            torch.cuda.reset_peak_memory_stats()


def build_device_memory_monitor() -> DeviceMemoryMonitor:
    mon = DeviceMemoryMonitor()
    logger.info(f"{mon.device_name} capacity: {mon.device_capacity_gib:.2f}GiB")
    return mon


class BaseLogger:
    def log(self, metrics: dict[str, Any], step: int) -> None:
        pass

    def close(self) -> None:
        pass


class TensorBoardLogger(BaseLogger):
    def __init__(self, log_dir: str, tag: str | None = None):
        from torch.utils.tensorboard import SummaryWriter

        self.tag = tag
        self.writer = SummaryWriter(log_dir, max_queue=1000)
        logger.info(f"TensorBoard logging enabled. Logs will be saved at {log_dir}")

    def log(self, metrics: dict[str, Any], step: int) -> None:
        for k, v in metrics.items():
            name = k if self.tag is None else f"{self.tag}/{k}"
            if isinstance(v, (list, tuple)) or (torch.is_tensor(v) and v.ndim > 0):
                self.writer.add_histogram(name, torch.as_tensor(v), step)
            else:
                self.writer.add_scalar(name, v, step)

    def close(self) -> None:
        self.writer.close()


class WandBLogger(BaseLogger):
    def __init__(self, log_dir: str, config_dict: dict[str, Any] | None = None, tag: str | None = None):
        import wandb

        self.wandb, self.tag = wandb, tag
        os.makedirs(log_dir, exist_ok=True)
        wandb.init(
            entity=os.getenv("WANDB_TEAM"), project=os.getenv("WANDB_PROJECT", "torchtitan"),
            name=os.getenv("WANDB_RUN_NAME"), id=os.getenv("WANDB_RUN_ID"), notes=os.getenv("WANDB_RUN_NOTES"),
            tags=os.getenv("WANDB_RUN_TAGS", "").split(",") if os.getenv("WANDB_RUN_TAGS") else None,
            group=os.getenv("WANDB_RUN_GROUP"), job_type=os.getenv("WANDB_RUN_JOB_TYPE"),
            resume_from=os.getenv("WANDB_RESUME_FROM"), fork_from=os.getenv("WANDB_FORK_FROM"),
            dir=log_dir, config=config_dict,
        )
        logger.info("WandB logging enabled")

    def log(self, metrics: dict[str, Any], step: int) -> None:
        self.wandb.log({(k if self.tag is None else f"{self.tag}/{k}"): v for k, v in metrics.items()}, step=step)

    def close(self) -> None:
        if self.wandb.run is not None:
            self.wandb.finish()


class LoggerContainer(BaseLogger):
    def __init__(self) -> None:
        self._loggers: list[BaseLogger] = []

    def add_logger(self, logger_instance: BaseLogger) -> None:
        self._loggers.append(logger_instance)

    def log(self, metrics: dict[str, Any], step: int) -> None:
        for lg in self._loggers:
            lg.log(metrics, step)

    @property
    def number_of_loggers(self) -> int:
        return len(self._loggers)

    def close(self) -> None:
        for lg in self._loggers:
            lg.close()


_V_SCHEDULES = ("ZBVZeroBubble", "DualPipeV")


def _get_metrics_rank(parallel_dims, pp_schedule: str = "1F1B") -> int:
    """Rank that owns the loss: rank 0 unless pipeline parallel, then the first rank of the last
    stage (for V-shaped schedules the last stage lives on pipeline rank 0)."""
    if not parallel_dims.pp_enabled or pp_schedule in _V_SCHEDULES:
        return 0
    return parallel_dims.world_size // parallel_dims.pp * (parallel_dims.pp - 1)


def ensure_pp_loss_visible(parallel_dims, pp_schedule: str, color) -> None:
    """Warn when LOG_RANK hides the rank(s) that print the loss under pipeline parallel."""
    if not parallel_dims.pp_enabled:
        return
    first = _get_metrics_rank(parallel_dims, pp_schedule)
    loss_ranks = set(range(first, first + parallel_dims.world_size // parallel_dims.pp)) if first else {0}
    visible = {int(r) for r in os.environ.get("LOG_RANK", "0").split(",") if r.strip()}
    if not (visible & loss_ranks):
        logger.warning(
            f"{color.red}Pipeline Parallel loss is not visible. Please add at least one rank of the last "
            f"stage (e.g. {first}) to LOG_RANK.{color.reset}"
        )


class MetricsProcessor(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        log_freq: int = 10
        enable_tensorboard: bool = False
        disable_color_printing: bool = False
        save_tb_folder: str = "tb"
        save_for_all_ranks: bool = False
        enable_wandb: bool = False
        log_moe_histogram: bool = True
        """*addition* log each MoE layer's token-per-expert histogram on logging steps."""

    def __init__(self, config: Config, *, parallel_dims, dump_folder: str = "./outputs", pp_schedule: str = "1F1B",
                 ft_enable: bool = False, ft_replica_id: int = 0, config_dict: dict[str, Any] | None = None,
                 tag: str | None = None, has_quantization: bool = False):
        self.config = config
        self.parallel_dims = parallel_dims
        self.logger = self._build_metric_logger(
            config=config, parallel_dims=parallel_dims, dump_folder=dump_folder, pp_schedule=pp_schedule,
            ft_enable=ft_enable, ft_replica_id=ft_replica_id, config_dict=config_dict, tag=tag,
        )
        self.device_memory_monitor = build_device_memory_monitor()
        self.color = utils.NoColor() if config.disable_color_printing else utils.Color()
        self.gpu_peak_flops = utils.get_peak_flops(self.device_memory_monitor.device_name)
        self.ntokens_since_last_log = 0
        self.data_loading_times: list[float] = []
        self.device_step_ms: list[float] = []
        self.time_last_log = time.perf_counter()
        self.device_memory_monitor.reset_peak_stats()
        self.has_quantization = has_quantization
        self.num_flops_per_token = -1
        self.optimizers = None
        self.lr_schedulers = None
        self.model_parts = None

    def should_log(self, step: int) -> bool:
        return step == 1 or step % self.config.log_freq == 0

    def _build_metric_logger(self, *, config, parallel_dims, dump_folder, pp_schedule, ft_enable=False,
                             ft_replica_id=0, config_dict=None, tag=None) -> BaseLogger:
        enabled = config.enable_tensorboard or config.enable_wandb
        rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
        if enabled and not config.save_for_all_ranks:
            enabled = rank == _get_metrics_rank(parallel_dims, pp_schedule)
        if not enabled:
            return BaseLogger()
        log_dir = os.path.join(dump_folder, config.save_tb_folder, datetime.now().strftime("%Y%m%d-%H%M"))
        if ft_enable:
            log_dir = os.path.join(log_dir, f"replica_{ft_replica_id}")
        if config.save_for_all_ranks:
            log_dir = os.path.join(log_dir, f"rank_{rank}")
        box = LoggerContainer()
        if config.enable_wandb:
            try:
                box.add_logger(WandBLogger(log_dir, config_dict=config_dict, tag=tag))
            except Exception as e:
                logger.error(f"Failed to create WandB logger: {e}")
        if config.enable_tensorboard:
            box.add_logger(TensorBoardLogger(log_dir, tag))
        return box

    def _moe_histograms(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        if not (self.config.log_moe_histogram and self.model_parts):
            return out
        for part in self.model_parts:
            layers = getattr(part, "layers", None)
            if layers is None:
                continue
            for name, block in layers.items():
                moe = getattr(block, "moe", None)
                if moe is not None and getattr(block, "moe_enabled", False):
                    t = moe.tokens_per_expert.detach().float().cpu()
                    out[f"moe/layer_{name}/tokens_per_expert"] = t.tolist()
                    mean = float(t.mean()) if t.numel() else 0.0
                    out[f"moe/layer_{name}/max_over_mean"] = float(t.max() / mean) if mean > 0 else 0.0
        return out

    def log(self, step: int, global_avg_loss: float, global_max_loss: float, grad_norm: float,
            extra_metrics: dict[str, Any] | None = None):
        assert self.num_flops_per_token > 0, "num_flops_per_token must be set"
        dt = time.perf_counter() - self.time_last_log
        tps = self.ntokens_since_last_log / (dt * self.parallel_dims.non_data_parallel_size)
        tflops = self.num_flops_per_token * tps / 1e12
        mfu = None if self.has_quantization else 100 * self.num_flops_per_token * tps / self.gpu_peak_flops
        n_load = max(len(self.data_loading_times), 1)
        mem = self.device_memory_monitor.get_peak_stats()
        metrics = {
            "loss_metrics/global_avg_loss": global_avg_loss,
            "loss_metrics/global_max_loss": global_max_loss,
            "grad_norm": grad_norm,
            "throughput(tps)": tps,
            "tflops": tflops,
            "time_metrics/end_to_end(s)": dt / self.config.log_freq,
            "time_metrics/data_loading(s)": sum(self.data_loading_times) / n_load,
            "time_metrics/data_loading(%)": 100 * sum(self.data_loading_times) / dt,
            "memory/max_active(GiB)": mem.max_active_gib,
            "memory/max_active(%)": mem.max_active_pct,
            "memory/max_reserved(GiB)": mem.max_reserved_gib,
            "memory/max_reserved(%)": mem.max_reserved_pct,
            "memory/num_alloc_retries": mem.num_alloc_retries,
            "memory/num_ooms": mem.num_ooms,
        }
        if mfu is not None:
            metrics["mfu(%)"] = mfu
        if self.device_step_ms:
            metrics["time_metrics/device_step(ms)"] = sum(self.device_step_ms) / len(self.device_step_ms)
        metrics.update(self._moe_histograms())
        if extra_metrics:
            metrics.update(extra_metrics)
        self.logger.log(metrics, step)
        c = self.color
        mfu_str = f"{mfu:.2f}%" if mfu is not None else "N/A"
        logger.info(
            f"{c.red}step: {step:2}  {c.green}loss: {global_avg_loss:8.5f}  {c.orange}grad_norm: {grad_norm:7.4f}  "
            f"{c.turquoise}memory: {mem.max_reserved_gib:5.2f}GiB({mem.max_reserved_pct:.2f}%)  "
            f"{c.blue}tps: {round(tps):,}  {c.cyan}tflops: {tflops:,.2f}  {c.magenta}mfu: {mfu_str}{c.reset}"
        )
        self.ntokens_since_last_log = 0
        self.data_loading_times.clear()
        self.device_step_ms.clear()
        self.time_last_log = time.perf_counter()
        self.device_memory_monitor.reset_peak_stats()

    def log_validation(self, loss: float, step: int, extra_metrics: dict[str, Any] | None = None):
        dt = time.perf_counter() - self.time_last_log
        mem = self.device_memory_monitor.get_peak_stats()
        tps = self.ntokens_since_last_log / (dt * self.parallel_dims.non_data_parallel_size)
        metrics = {
            "validation_metrics/loss": loss,
            "validation_metrics/throughput(tps)": tps,
            "validation_metrics/memory/max_active(GiB)": mem.max_active_gib,
            "validation_metrics/memory/max_active(%)": mem.max_active_pct,
            "validation_metrics/memory/max_reserved(GiB)": mem.max_reserved_gib,
            "validation_metrics/memory/max_reserved(%)": mem.max_reserved_pct,
        }
        if extra_metrics:
            metrics.update(extra_metrics)
        self.logger.log(metrics, step)
        c = self.color
        logger.info(
            f"{c.yellow}validate step: {step:2}  {c.green}loss: {loss:7.4f}  "
            f"{c.turquoise}memory: {mem.max_reserved_gib:5.2f}GiB({mem.max_reserved_pct:.2f}%)  "
            f"{c.blue}tps: {round(tps):,}{c.reset}"
        )
        self.ntokens_since_last_log = 0
        self.time_last_log = time.perf_counter()
        self.device_memory_monitor.reset_peak_stats()

    def close(self):
        self.logger.close()
