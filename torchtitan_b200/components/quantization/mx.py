"""MXFP8 training converter (``mxfp8_rceil``): every module whose fqn contains one of ``fqns`` --
``Linear`` layers and routed-expert grouped GEMMs -- quantises both GEMM operands to e4m3 with one
E8M0 scale per 32 elements along the contraction dimension, in all three passes. Token groups are
padded to 32 rows unless the dispatcher already aligns them.
Parity: torchtitan/components/quantization/mx.py:26-140. Needs sm_100 (block-scaled tensor-core MMA)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, Literal

import torch
import torch.nn as nn

from torchtitan_b200.ops.quant import QuantRecipe
from torchtitan_b200.tools.logging import logger

from . import MXFP8_GROUP_ALIGNMENT_SIZE, QuantizationConverter


class MXFP8Converter(QuantizationConverter):
    @dataclass(kw_only=True, slots=True)
    class Config(QuantizationConverter.Config):
        _quantization_type: ClassVar[str] = "mxfp8"
        recipe_name: Literal["mxfp8_rceil"] = "mxfp8_rceil"
        fqns: list[str] = field(default_factory=list)
        pad_token_groups_for_grouped_mm: bool = True
        emulate: bool = False

    def __init__(self, config: Config, *, parallel_dims, model_compile_enabled: bool = False):
        self.enabled = False
        on_sm100 = torch.cuda.is_available() and torch.cuda.get_device_capability() >= (10, 0)
        assert on_sm100 or config.emulate, "MXFP8 is only supported on SM100 or architectures"
        self.config = config
        self.recipe = QuantRecipe(kind="mxfp8", scaling="block32", emulate=config.emulate,
                                  pad_token_groups=config.pad_token_groups_for_grouped_mm)
        self.enabled = True
        logger.info("MXFP8 MoE training enabled")

    def convert(self, model: nn.Module):
        if not self.enabled:
            return
        from torchtitan_b200.models.common.moe.moe import GroupedExperts

        n = 0
        for fqn, mod in model.named_modules():
            if not any(t in fqn for t in self.config.fqns):
                continue
            if isinstance(mod, GroupedExperts):
                mod.quant = self.recipe
                if self.config.pad_token_groups_for_grouped_mm and hasattr(mod.dispatcher, "alignment"):
                    from torchtitan_b200.models.common.moe.moe import group_alignment

                    # 32 rows for the definition; 128 where the native grouped kernel runs (its scale chunks cover
                    # 128 rows). Dispatchers installed later by expert parallelism ask group_alignment() again.
                    mod.dispatcher.alignment = group_alignment(mod, MXFP8_GROUP_ALIGNMENT_SIZE)
                n += 1
            elif isinstance(mod, nn.Linear) and mod.weight.shape[0] % 32 == 0 and mod.weight.shape[1] % 32 == 0:
                mod.quant = self.recipe
                n += 1
        logger.info(f"Converted {n} layers matching FQNS {self.config.fqns} to use dynamic {self.config.recipe_name} "
                    "quantization for grouped_mm and linear ops")

    def post_optimizer_hook(self, model: nn.Module | list[nn.Module]):
        return
