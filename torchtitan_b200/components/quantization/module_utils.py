"""Helpers for model converters that replace modules by instances of other classes.

The converters of this framework keep every layer's class and attach a recipe to it (``Linear.quant``), so they need
none of this. A user-written converter that swaps ``nn.Linear`` layers for a library's own class (as torchao's
``Float8Linear`` / ``MXLinear`` conversions do in the reference, torchtitan/components/quantization/module_utils.py:21-113)
loses two things: instance attributes of the old objects, and the ``Module`` protocol (``init_weights``, ``Config``) the
trainer relies on. These functions save the attributes by fully-qualified name, give the swapped objects a class that
also derives from a ``Module`` subclass, and check that no layer was missed.
"""

from __future__ import annotations

from typing import Any

import torch.nn as nn

from torchtitan_b200.protocols.module import Module

__all__ = ["capture_module_attrs", "inject_module_protocol", "verify_module_protocol"]


def capture_module_attrs(model: nn.Module, attr_names: list[str], nn_module_cls: type[nn.Module] = nn.Linear) -> dict[str, dict[str, Any]]:
    """``{fqn: {attribute: value}}`` for every ``nn_module_cls`` instance that has all of ``attr_names``."""
    saved = {}
    for fqn, mod in model.named_modules():
        if isinstance(mod, nn_module_cls) and all(hasattr(mod, a) for a in attr_names):
            saved[fqn] = {a: getattr(mod, a) for a in attr_names}
    return saved


def inject_module_protocol(model: nn.Module, module_cls: type[Module], saved_attrs: dict[str, dict[str, Any]] | None = None,
                           nn_module_cls: type[nn.Module] = nn.Linear) -> None:
    """Every ``nn_module_cls`` instance that is not a ``Module`` yet gets a class deriving from its own class and from
    ``module_cls`` (one such class per original class; it cannot be constructed directly), and the attributes saved for
    its name are put back."""
    mixed: dict[type, type] = {}

    def _no_constructor(self, *args, **kwargs):
        raise RuntimeError(f"{type(self).__name__} is a patched class created by inject_module_protocol and should not be "
                           "constructed directly.")

    for fqn, mod in model.named_modules():
        if not isinstance(mod, nn_module_cls) or isinstance(mod, Module):
            continue
        cls = type(mod)
        if cls not in mixed:
            mixed[cls] = type(f"{cls.__name__}_With{module_cls.__name__}", (cls, module_cls), {"__init__": _no_constructor})
        mod.__class__ = mixed[cls]
        for name, value in (saved_attrs or {}).get(fqn, {}).items():
            setattr(mod, name, value)


def verify_module_protocol(model: nn.Module, target_cls: type[nn.Module], module_cls: type[Module] = Module) -> None:
    """Raise when an instance of ``target_cls`` is not also a ``module_cls``."""
    missed = [(fqn, type(mod).__name__) for fqn, mod in model.named_modules()
              if isinstance(mod, target_cls) and not isinstance(mod, module_cls)]
    if missed:
        listing = ", ".join(f"'{fqn}' ({name})" for fqn, name in missed)
        raise RuntimeError(f"The following {target_cls.__name__} modules do not satisfy {module_cls.__name__} protocol: {listing}")
