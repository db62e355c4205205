"""Module filter shared by the float8 and MXFP8 converters
(torchtitan/components/quantization/utils.py:10-28): only ``nn.Linear`` with both dimensions
divisible by 16 and a name matching none of ``filter_fqns`` is converted."""

import torch.nn as nn


def module_filter_fn(mod: nn.Module, fqn: str, filter_fqns: list[str]) -> bool:
    if not isinstance(mod, nn.Linear):
        return False
    ok_dims = mod.weight.shape[0] % 16 == 0 and mod.weight.shape[1] % 16 == 0
    return ok_dims and not any(f in fqn for f in filter_fqns)
