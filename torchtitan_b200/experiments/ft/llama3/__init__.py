"""Llama 3 under the fault-tolerant trainer: the family's own model specification
(torchtitan/experiments/ft/llama3/__init__.py)."""

from torchtitan_b200.models.llama3 import model_registry  # noqa: F401

__all__ = ["model_registry"]
