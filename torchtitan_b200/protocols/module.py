"""``Module`` = ``nn.Module`` + ``Configurable`` with an ``init_weights`` contract.

Parity: torchtitan/protocols/module.py:12-23.
"""

import torch.nn as nn

from torchtitan_b200.config.configurable import Configurable


class Module(nn.Module, Configurable):
    """Base of every model building block. ``init_weights`` must be callable on a module
    whose parameters were just materialised with ``to_empty`` (built on ``meta``). The default does nothing, which suits
    modules without learnable parameters or with weights loaded from elsewhere; modules with parameters override it."""

    def init_weights(self, **kwargs) -> None:
        return None
