"""Activation checkpointing under the reference's module name (torchtitan/distributed/activation_checkpoint.py)."""

from torchtitan_b200.parallel.ac import apply_ac, default_op_sac_save_list  # noqa: F401

__all__ = ["apply_ac", "default_op_sac_save_list"]
