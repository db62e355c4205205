"""``Configurable``: every component owns a nested ``Config`` dataclass that can build it.

Behavioural parity with torchtitan/config/configurable.py:14-180:

* ``Config`` must be declared ``@dataclass(kw_only=True, slots=True)``; the check runs
  when the *outer* class is created because ``slots=True`` makes ``@dataclass`` return a
  new class object.
* ``cfg.build(**kw)``: when every keyword names a config field the values are folded into
  a clone of the config (conflicts with already-set values raise ``ValueError``); when no
  keyword names a field they are forwarded to the owner's ``__init__``; a mixture raises
  ``TypeError``.
* fields declared ``field(init=False)`` are slots that only ``build()`` fills; an unfilled
  slot raises ``TypeError`` at build time and prints as ``<UNSET>`` in ``repr``.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, ClassVar

import torch

_MISSING = object()


def _same(a: Any, b: Any) -> bool:
    if isinstance(a, torch.Tensor) or isinstance(b, torch.Tensor):
        return (
            isinstance(a, torch.Tensor)
            and isinstance(b, torch.Tensor)
            and a.shape == b.shape
            and bool(torch.equal(a, b))
        )
    return a == b


class Configurable:
    @dataclass(kw_only=True, slots=True)
    class Config:
        """Base of every component config. Use :meth:`to_dict`, not ``dataclasses.asdict``,
        because late-bound slots may still be empty."""

        _owner: ClassVar[type | None] = None

        # -- introspection that tolerates empty late-bound slots -----------------
        def _items(self):
            for f in dataclasses.fields(self):
                yield f, getattr(self, f.name, _MISSING)

        def __repr__(self) -> str:
            body = ", ".join(
                f"{f.name}=<UNSET>" if v is _MISSING else f"{f.name}={v!r}"
                for f, v in self._items()
            )
            return f"{type(self).__name__}({body})"

        def to_dict(self) -> dict:
            out: dict[str, Any] = {}
            for f, v in self._items():
                if v is _MISSING:
                    continue
                if hasattr(v, "to_dict"):
                    out[f.name] = v.to_dict()
                elif dataclasses.is_dataclass(v) and not isinstance(v, type):
                    out[f.name] = dataclasses.asdict(v)
                elif isinstance(v, (list, tuple)):
                    out[f.name] = [
                        x.to_dict() if hasattr(x, "to_dict") else x for x in v
                    ]
                else:
                    out[f.name] = v
            return out

        # -- build ------------------------------------------------------------------
        def _clone_filled(self, **late):
            clone = dataclasses.replace(self)
            for f, v in self._items():
                if f.init:
                    continue
                if f.name in late:
                    setattr(clone, f.name, late[f.name])
                elif v is not _MISSING:
                    setattr(clone, f.name, v)
                else:
                    raise TypeError(
                        f"{type(self).__name__} field '{f.name}' (init=False) "
                        "was not provided via build()"
                    )
            return clone

        def build(self, **kwargs):
            owner = type(self)._owner
            if owner is None:
                raise NotImplementedError(
                    f"{type(self).__name__} has no owner class. "
                    "Define Config inside a Configurable subclass."
                )
            names = {f.name for f in dataclasses.fields(self)}
            as_fields = {k for k in kwargs if k in names}
            as_ctor = set(kwargs) - as_fields
            if as_fields and as_ctor:
                raise TypeError(
                    f"{type(self).__name__}.build() kwargs must either all be config "
                    f"fields or all be constructor arguments; got fields "
                    f"{sorted(as_fields)} mixed with {sorted(as_ctor)}"
                )
            if as_fields:
                for k in as_fields:
                    cur = getattr(self, k, _MISSING)
                    if cur is not _MISSING and not _same(cur, kwargs[k]):
                        raise ValueError(
                            f"{type(self).__name__}.build() conflict for '{k}': "
                            f"config has {cur!r} but got {kwargs[k]!r}"
                        )
                init_over = {
                    k: v
                    for k, v in kwargs.items()
                    if any(f.name == k and f.init for f in dataclasses.fields(self))
                }
                late = {k: v for k, v in kwargs.items() if k not in init_over}
                clone = self._clone_filled(**late)
                for k, v in init_over.items():
                    setattr(clone, k, v)
                return owner(config=clone)
            return owner(config=self._clone_filled(), **kwargs)

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        cfg = cls.__dict__.get("Config")
        if cfg is None or not (
            isinstance(cfg, type) and issubclass(cfg, Configurable.Config)
        ):
            return
        if "__slots__" not in cfg.__dict__:
            raise TypeError(
                f"{cls.__name__}.Config must use @dataclass(kw_only=True, slots=True)"
            )
        for f in dataclasses.fields(cfg):
            if f.init and not f.kw_only:
                raise TypeError(
                    f"{cls.__name__}.Config field '{f.name}' must be keyword-only"
                )
        cfg.__repr__ = Configurable.Config.__repr__
        cfg._owner = cls
