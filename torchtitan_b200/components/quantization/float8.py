"""placeholder"""
from dataclasses import dataclass, field
from torchtitan_b200.config.configurable import Configurable
class Float8LinearConverter(Configurable):
    _quantization_type = "float8"
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        enable_fsdp_float8_all_gather: bool = False
        precompute_float8_dynamic_scale_for_fsdp: bool = False
        recipe_name: str | None = None
        filter_fqns: list[str] = field(default_factory=list)
        emulate: bool = False
    def __init__(self, config, *, parallel_dims, model_compile_enabled=False):
        self.config = config
    def convert(self, model): pass
    def post_optimizer_hook(self, model): pass
