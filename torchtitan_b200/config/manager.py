"""``ConfigManager``: ``--module M --config fn`` picks a Python function that returns a full
job config; the remaining ``--section.key value`` flags override it through tyro.

Parity: torchtitan/config/manager.py:19-44 (precedence CLI > registry function), :46-151
(short module names are searched under ``models`` then ``experiments``; any other value is
treated as a fully-qualified module path, with or without ``.config_registry``), :222-235
(``list[str]`` accepts ``A,B,C``), :242-271 (``python -m …config.manager`` prints the config).
"""

from __future__ import annotations

import contextlib
import dataclasses
import importlib
import os
import sys

import tyro

from torchtitan_b200.tools.logging import logger

_PKG = "torchtitan_b200"

custom_registry = tyro.constructors.ConstructorRegistry()


@custom_registry.primitive_rule
def _comma_list(type_info: tyro.constructors.PrimitiveTypeInfo):
    if type_info.type != list[str]:
        return None
    return tyro.constructors.PrimitiveConstructorSpec(
        nargs=1,
        metavar="A,B,C,...",
        instance_from_str=lambda a: a[0].split(","),
        is_instance=lambda v: isinstance(v, list) and all(isinstance(i, str) for i in v),
        str_from_instance=lambda v: [",".join(v)],
    )


def _pop_flag(args: list[str], flag: str) -> tuple[str | None, list[str]]:
    value, rest, i = None, [], 0
    while i < len(args):
        a = args[i]
        if a == flag:
            if i + 1 >= len(args):
                raise ValueError(f"{flag} requires a value")
            value = args[i + 1]
            i += 2
            continue
        if a.startswith(flag + "="):
            value = a[len(flag) + 1 :]
        else:
            rest.append(a)
        i += 1
    return value, rest


@contextlib.contextmanager
def _distinct_element_names(config):
    """While the command line is parsed, the element types of a heterogeneous list in the configuration carry distinct
    class names. The parser offers the element types of a list such as ``model_converters.converters`` as alternatives
    named after their classes; the nested ``Config`` classes of two converters are both called ``Config``, which it cannot
    tell apart (a job configuration with a float8 linear converter and a float8 grouped-GEMM converter then fails to
    parse at all). ``Float8LinearConverter.Config`` becomes ``Float8LinearConverterConfig`` for the duration."""
    renamed: list[tuple[type, str]] = []

    def walk(obj, depth=0):
        if depth > 8 or not dataclasses.is_dataclass(obj) or isinstance(obj, type):
            return
        for f in dataclasses.fields(obj):
            value = getattr(obj, f.name, None)
            if isinstance(value, (list, tuple)):
                types = {type(v) for v in value if dataclasses.is_dataclass(v)}
                names = [t.__name__ for t in types]
                for t in types:
                    if names.count(t.__name__) > 1:
                        renamed.append((t, t.__name__))
                        t.__name__ = t.__qualname__.replace(".", "")
                for v in value:
                    walk(v, depth + 1)
            else:
                walk(value, depth + 1)

    walk(config)
    try:
        yield
    finally:
        for t, name in renamed:
            t.__name__ = name


class ConfigManager:
    def __init__(self):
        self.config = None

    @staticmethod
    def register_tyro_rules(registry) -> None:  # kept for API compatibility
        return None

    def parse_args(self, args: list[str] | None = None):
        args = list(sys.argv[1:] if args is None else args)
        loaded, rest = self._load_config(args)
        with _distinct_element_names(loaded):
            self.config = tyro.cli(
                type(loaded), args=rest, default=loaded, registry=custom_registry
            )
        self._validate_config()
        return self.config

    def _load_config(self, args: list[str]):
        module_name, args = _pop_flag(args, "--module")
        config_name, args = _pop_flag(args, "--config")
        example = "Example: --module llama3 --config llama3_debugmodel"
        if module_name is None:
            raise ValueError(f"--module is required. {example}")
        if config_name is None:
            raise ValueError(f"--config is required. {example}")

        from torchtitan_b200.experiments import _supported_experiments
        from torchtitan_b200.models import _supported_models

        known = _supported_models | _supported_experiments
        if module_name in known:
            candidates = [
                f"{_PKG}.models.{module_name}.config_registry",
                f"{_PKG}.experiments.{module_name}.config_registry",
            ]
        else:
            candidates = [f"{module_name}.config_registry", module_name]
        module, path, last_err = None, None, None
        for cand in candidates:
            try:
                module = importlib.import_module(cand)
                path = cand
                break
            except ModuleNotFoundError as e:
                # only swallow "this candidate does not exist"; real import errors inside
                # an existing registry must surface.
                if e.name is None or not cand.startswith(e.name):
                    raise
                last_err = e
        if module is None:
            raise ImportError(
                f"Cannot import module '{module_name}' (no config registry found for it). "
                f"Supported short names: {sorted(known)}"
            ) from last_err
        fn = getattr(module, config_name, None)
        if fn is None or not callable(fn):
            avail = sorted(
                n
                for n in dir(module)
                if not n.startswith("_") and n[0].islower() and callable(getattr(module, n))
            )
            raise ValueError(
                f"Config function '{config_name}' not found in {path}. "
                f"Available config functions: {avail}"
            )
        return fn(), args

    def _validate_config(self) -> None:
        path = getattr(self.config, "hf_assets_path", None)
        if path is None:
            return
        if path.endswith("tokenizer.model"):
            raise ValueError(
                "hf_assets_path must be a directory with tokenizer.json, not tokenizer.model"
            )
        if not os.path.exists(path):
            logger.warning(f"HF assets path {path} does not exist!")


if __name__ == "__main__":
    from rich import print as rprint
    from rich.pretty import Pretty

    rprint(Pretty(ConfigManager().parse_args()))
