"""Reshard-after-forward policy. Parity: torchtitan/distributed/fsdp.py:8-32 ("default" =
reshard unless pipeline parallel, where gathered parameters would be re-fetched per
micro-batch; "always"; "never"). B200 twist: under "default", when the whole compute copy of
the model fits in a small fraction of the GPU's memory the gathered parameters are kept between
forward and backward, which removes one all-gather per unit per step."""

from __future__ import annotations

import torch

KEEP_GATHERED_FRACTION = 0.15


def get_fsdp_reshard_after_forward_policy(policy: str, pp_enabled: bool, *, param_bytes: int | None = None) -> bool:
    if policy == "always":
        return True
    if policy == "never":
        return False
    if policy == "default":
        if pp_enabled:
            return False
        if param_bytes is not None and torch.cuda.is_available():
            total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
            if param_bytes <= KEEP_GATHERED_FRACTION * total:
                return False
        return True
    raise ValueError(f"Invalid reshard_after_forward_policy: {policy}. Allowed values are 'default', 'always', or 'never'.")
