"""The reference's module name for the permutation-index helpers (torchtitan/models/common/moe/kernels.py:71-218);
the code lives in ``permute.py``."""

from .permute import fill_indices, fill_indices_cpu, fill_indices_wrapper, generate_permute_indices

__all__ = ["fill_indices", "fill_indices_cpu", "fill_indices_wrapper", "generate_permute_indices"]
