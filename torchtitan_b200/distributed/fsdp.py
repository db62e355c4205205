"""FSDP policy helper under the reference's module name (torchtitan/distributed/fsdp.py); the runtime itself is
``torchtitan_b200.parallel.fsdp``."""

from torchtitan_b200.parallel.fsdp_policy import get_fsdp_reshard_after_forward_policy  # noqa: F401

__all__ = ["get_fsdp_reshard_after_forward_policy"]
