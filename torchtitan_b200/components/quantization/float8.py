"""Float8 training converters.

Parity: torchtitan/components/quantization/float8.py:35-330 -- ``Float8LinearConverter`` (recipes
``tensorwise`` (default), ``rowwise``, ``rowwise_with_gw_hp``; ``filter_fqns`` with the
``auto_filter_small_kn`` flag that skips layers too small to profit; ``emulate`` for hardware
without float8; float8 all-gather and scale precompute options for tensorwise + FSDP) and
``Float8GroupedMMConverter`` (routed experts whose fqn contains one of ``fqns``; token groups
aligned to 16 rows)."""

from __future__ import annotations

from dataclasses import dataclass, field
from functools import partial
from typing import ClassVar, Literal

import torch
import torch.nn as nn

from torchtitan_b200.ops.quant import QuantRecipe
from torchtitan_b200.tools.logging import logger

from . import FP8_GROUP_ALIGNMENT_SIZE, QuantizationConverter
from .utils import module_filter_fn

AUTO_FILTER_SMALL_KN_FLAG = "auto_filter_small_kn"


def _auto_filter(mod: nn.Module, fqn: str, recipe: str, filter_fqns: list[str]) -> bool:
    """Skip layers whose (K, N) is too small for the quantise overhead to pay off (thresholds of the
    float8 documentation: tensorwise needs K,N >= ~(4096,1024)/(2048,4096)..., rowwise larger)."""
    if not module_filter_fn(mod, fqn, filter_fqns):
        return False
    n, k = mod.weight.shape
    if recipe == "tensorwise":
        small = (k <= 4096 and n <= 1024) or (k <= 2048 and n <= 2048) or (k <= 1024 and n <= 4096)
    else:
        small = (k <= 2048 and n <= 4096) or (k <= 4096 and n <= 2048)
    return not small


def _has_fp8_hardware() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability() >= (8, 9)


class Float8LinearConverter(QuantizationConverter):
    @dataclass(kw_only=True, slots=True)
    class Config(QuantizationConverter.Config):
        _quantization_type: ClassVar[str] = "float8"
        enable_fsdp_float8_all_gather: bool = False
        precompute_float8_dynamic_scale_for_fsdp: bool = False
        recipe_name: Literal["tensorwise", "rowwise", "rowwise_with_gw_hp"] | None = None
        filter_fqns: list[str] = field(default_factory=list)
        emulate: bool = False

    def __init__(self, config: Config, *, parallel_dims, model_compile_enabled: bool = False):
        self.enabled = False
        if not (_has_fp8_hardware() or (config.emulate and not model_compile_enabled)):
            raise ValueError(
                "Failed to swap to Float8Linear because float8 is only supported on SM89 or later."
                "To enable testing on older hardware, set `float8.emulate` to True in eager mode."
            )
        filter_fqns = list(config.filter_fqns)
        recipe = config.recipe_name or "tensorwise"
        if AUTO_FILTER_SMALL_KN_FLAG in filter_fqns:
            filter_fqns.remove(AUTO_FILTER_SMALL_KN_FLAG)
            self.filter_fn = partial(_auto_filter, recipe=recipe, filter_fqns=filter_fqns)
        else:
            self.filter_fn = partial(module_filter_fn, filter_fqns=filter_fqns)
        self.filter_fqns = filter_fqns
        if config.recipe_name is not None:
            assert not config.enable_fsdp_float8_all_gather, (
                "using `float8_config.enable_fsdp_float8_all_gather` together with `float8_config.recipe_name` is not supported"
            )
            self.fp8_all_gather = self.precompute_scale = False
            logger.info(f"Float8 training active with recipe {config.recipe_name}")
        else:
            self.fp8_all_gather = parallel_dims.dp_shard_enabled and config.enable_fsdp_float8_all_gather
            self.precompute_scale = self.fp8_all_gather and config.precompute_float8_dynamic_scale_for_fsdp
            logger.info("Float8 tensorwise scaled training active")
            if self.fp8_all_gather:
                # said at start-up: the FSDP runtime gathers the bf16 compute copy of a shard (written by the fused
                # AdamW in the same pass as the fp32 master) and the linears quantise after the gather
                logger.warning("float8.enable_fsdp_float8_all_gather has no effect in this runtime: parameters are gathered "
                               "in bf16 (the gather of the next unit runs on a side stream behind the current unit's compute); "
                               "precompute_float8_dynamic_scale_for_fsdp is ignored with it")
        self.recipe = QuantRecipe(kind="float8", scaling=recipe, emulate=config.emulate)
        self.enabled = True

    def convert(self, model: nn.Module):
        if not self.enabled:
            return
        n = 0
        for fqn, mod in model.named_modules():
            if self.filter_fn(mod, fqn):
                mod.quant = self.recipe
                n += 1
        logger.info(f"Float8 ({self.recipe.scaling}) enabled on {n} linear layers, float8 all-gather={self.fp8_all_gather}")

    def post_optimizer_hook(self, model: nn.Module | list[nn.Module]):
        """The reference refreshes every converted weight's amax here for its float8 all-gather
        (torchtitan/components/quantization/float8.py:104-128). Parameters are gathered in bf16 in this runtime and
        each linear takes the amax of the gathered weight when it quantises, so there is nothing to precompute."""
        return


class Float8GroupedMMConverter(QuantizationConverter):
    @dataclass(kw_only=True, slots=True)
    class Config(QuantizationConverter.Config):
        _quantization_type: ClassVar[str] = "float8"
        fqns: list[str] | str = field(default_factory=list)

    def __init__(self, config: Config, *, parallel_dims, model_compile_enabled: bool = False):
        self.enabled = False
        self.fqns = [config.fqns] if isinstance(config.fqns, str) else list(config.fqns)
        if not _has_fp8_hardware():
            raise ValueError("Float8 MoE training only supported on SM89 or later.")
        self.recipe = QuantRecipe(kind="float8", scaling="rowwise")
        self.enabled = True
        logger.info("Float8 MoE training enabled")

    def convert(self, model: nn.Module):
        if not self.enabled:
            return
        from torchtitan_b200.models.common.moe.moe import GroupedExperts

        for fqn, mod in model.named_modules():
            if isinstance(mod, GroupedExperts) and any(t in fqn for t in self.fqns):
                mod.quant = self.recipe
                if hasattr(mod.dispatcher, "alignment"):
                    mod.dispatcher.alignment = FP8_GROUP_ALIGNMENT_SIZE
        logger.info(f"Converted MoE layers matching FQNS {self.fqns} to use dynamic float8 rowwise quantization with scaled grouped GEMMs")

    def post_optimizer_hook(self, model: nn.Module | list[nn.Module]):
        return


def find_float8_linear_config(converters: list) -> "Float8LinearConverter.Config | None":
    """The single Float8LinearConverter config of a converter list, or None."""
    found = [c for c in converters if isinstance(c, Float8LinearConverter.Config)]
    if len(found) > 1:
        raise ValueError("Only one Float8LinearConverter is supported")
    return found[0] if found else None
