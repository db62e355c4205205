from .moe import MoE, GroupedExperts, TokenChoiceTopKRouter, TokenReorderer
from .permute import fill_indices_cpu, generate_permute_indices

__all__ = [
    "MoE",
    "GroupedExperts",
    "TokenChoiceTopKRouter",
    "TokenReorderer",
    "fill_indices_cpu",
    "generate_permute_indices",
]
