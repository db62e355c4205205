"""Small runtime helpers: device discovery, GC scheduling, peak-FLOPs table, colours.

Parity: torchtitan/tools/utils.py:21-256.
"""

from __future__ import annotations

import contextlib
import gc
import time
from dataclasses import dataclass

import torch

from .logging import logger


def has_cuda_capability(major: int, minor: int) -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability() >= (major, minor)


def is_sm100() -> bool:
    """True when the current device can run this framework's sm_100a kernels."""
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10


def get_device_info() -> tuple[str, object]:
    """('cuda', torch.cuda) when a GPU is present, else ('cpu', torch.cpu).

    Unlike the reference (tools/utils.py:36-42, which falls back to 'cuda' on a host with no
    accelerator) the CPU answer is real, so the Trainer also runs on gloo-only hosts.
    """
    if torch.cuda.is_available():
        return "cuda", torch.cuda
    return "cpu", torch.cpu


device_type, device_module = get_device_info()


class GarbageCollection:
    """Python's GC is switched off and run by hand every ``gc_freq`` steps so that all ranks
    pause at the same step instead of at random ones."""

    def __init__(self, gc_freq: int = 1000, debug: bool = False):
        assert gc_freq > 0, "gc_freq must be a positive integer"
        self.gc_freq = gc_freq
        self.debug = debug
        gc.disable()
        self.collect("Initial GC collection")
        if debug:
            from torch.utils.viz._cycles import warn_tensor_cycles

            if (not torch.distributed.is_initialized()) or torch.distributed.get_rank() == 0:
                warn_tensor_cycles()

    def run(self, step_count: int) -> None:
        if self.debug:
            self.collect("Force GC to perform collection to obtain debug information")
            gc.collect()
        elif step_count > 1 and step_count % self.gc_freq == 0:
            self.collect("Performing periodic GC collection")

    @staticmethod
    def collect(reason: str, generation: int = 1) -> None:
        t0 = time.monotonic()
        gc.collect(generation)
        logger.info("[GC] %s took %.2f seconds", reason, time.monotonic() - t0)


# dense bf16 tensor-core peaks in FLOP/s, keyed by substrings of the device name
_PEAKS = (
    ("GB200", 2.5e15),
    ("B200", 2.25e15),
    ("H200", 989e12),
    ("H100 NVL", 835e12),
    ("H100 PCIe", 756e12),
    ("H100", 989e12),
    ("A100", 312e12),
    ("MI355X", 2500e12),
    ("MI325X", 1300e12),
    ("MI300X", 1300e12),
    ("MI250X", 191.5e12),
    ("l40s", 362e12),
)


def get_peak_flops(device_name: str) -> float:
    """Nominal dense bf16 peak used for MFU (B200 = 2.25e15, torchtitan/tools/utils.py:122-124)."""
    for key, val in _PEAKS:
        if key.lower() in device_name.lower():
            return val
    logger.warning(f"Peak flops undefined for: {device_name}, fallback to A100")
    return 312e12


@dataclass(frozen=True)
class Color:
    black: str = "\033[30m"
    red: str = "\033[31m"
    green: str = "\033[32m"
    yellow: str = "\033[33m"
    blue: str = "\033[34m"
    magenta: str = "\033[35m"
    cyan: str = "\033[36m"
    white: str = "\033[37m"
    reset: str = "\033[39m"
    orange: str = "\033[38;2;180;60;0m"
    turquoise: str = "\033[38;2;54;234;195m"


@dataclass(frozen=True)
class NoColor:
    black: str = ""
    red: str = ""
    green: str = ""
    yellow: str = ""
    blue: str = ""
    magenta: str = ""
    cyan: str = ""
    white: str = ""
    reset: str = ""
    orange: str = ""
    turquoise: str = ""


@contextlib.contextmanager
def set_default_dtype(dtype: torch.dtype):
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        yield
    finally:
        torch.set_default_dtype(old)


def _round_up(x: int, y: int) -> int:
    return ((x + y - 1) // y) * y


def check_if_feature_in_pytorch(feature_name: str, pull_request: str, min_nightly_version: str | None = None) -> None:
    if "git" in torch.__version__:
        logger.warning(
            f"detected that the pytorch is built from source. Please make sure the PR "
            f"({pull_request}) is included in pytorch for correct {feature_name}."
        )
    elif min_nightly_version is not None and torch.__version__ < min_nightly_version:
        logger.warning(
            f"detected that the pytorch version {torch.__version__} is older than "
            f"{min_nightly_version}. Please upgrade to get {feature_name}."
        )
