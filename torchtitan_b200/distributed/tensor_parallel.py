"""Tensor parallel under the reference's module name (torchtitan/distributed/tensor_parallel.py)."""

from torchtitan_b200.parallel.tp import apply_tp_to_decoder  # noqa: F401

__all__ = ["apply_tp_to_decoder"]
