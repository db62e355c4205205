"""Quantised-training converters (float8 and MXFP8). A converter does not swap module classes: it
attaches a :class:`~torchtitan_b200.ops.quant.QuantRecipe` to the selected ``Linear`` /
``GroupedExperts`` modules, whose forward then routes through the quantised GEMM path; parameter
names, init attributes and the state dict stay exactly as before.
Parity: torchtitan/components/quantization/__init__.py (alignment constants, converter base class)."""

from dataclasses import dataclass
from typing import ClassVar

from torchtitan_b200.config.configurable import Configurable

FP8_GROUP_ALIGNMENT_SIZE = 16
MXFP8_GROUP_ALIGNMENT_SIZE = 32


class QuantizationConverter(Configurable):
    """Base of every quantisation converter (identified with ``isinstance``)."""

    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        _quantization_type: ClassVar[str]
