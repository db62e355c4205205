"""Expert parallel under the reference's module name (torchtitan/distributed/expert_parallel.py). The reference
expresses expert parallel as DTensor ``ParallelStyle`` classes; here the token exchange lives in dispatcher objects that
``apply_moe_ep_tp`` installs on the experts (``parallel/ep.py``, ``parallel/nvlink_ep.py``)."""

from torchtitan_b200.parallel.ep import AllToAllDispatcher, all_to_all_rows, apply_moe_ep_tp  # noqa: F401

__all__ = ["AllToAllDispatcher", "all_to_all_rows", "apply_moe_ep_tp"]
