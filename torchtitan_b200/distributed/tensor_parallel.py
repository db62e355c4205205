"""Tensor parallel under the reference's module name (torchtitan/distributed/tensor_parallel.py)."""

from torchtitan_b200.parallel.tp import apply_tp_to_decoder  # noqa: F401

__all__ = ["apply_tp_to_decoder", "maybe_enable_async_tp"]


def maybe_enable_async_tp(parallelism, compile_config, tp_mesh) -> None:
    """Kept for call sites written against the reference, where this switches on a compiler pass
    (tensor_parallel.py:20-45). Here asynchronous tensor parallel is a property of the sharded layers:
    ``apply_tp_to_decoder(..., async_tp=parallelism.enable_async_tensor_parallel)`` installs the fused all-gather -> GEMM
    and GEMM -> reduce-scatter kernels, and needs no compiler."""
    if getattr(parallelism, "enable_async_tensor_parallel", False):
        from torchtitan_b200.tools.logging import logger

        logger.info("Async TP is enabled")
