"""Splitting a decoder into fragments for streaming DiLoCo: either by explicit module names or evenly by layers, with
the embedding going to the first fragment and final norm + output to the last (the same rule as pipeline stage splits).
Parity: torchtitan/experiments/ft/diloco/utils.py:14-135."""

from __future__ import annotations

import torch.nn as nn

from torchtitan_b200.parallel.pp import generate_llm_fqn_per_model_part


class _Fragment(nn.Module):
    """A view over some sub-modules of a model (shares their parameters)."""

    def __init__(self, model: nn.Module, names: list[str]):
        super().__init__()
        self.names = names
        for n in names:
            self.add_module(n.replace(".", "_"), model.get_submodule(n))


def module_split(model: nn.Module, module_fqns_per_model_fragment: list[list[str]]) -> list[nn.Module]:
    return [_Fragment(model, names) for names in module_fqns_per_model_fragment]


def fragment_llm(model: nn.Module, ft_config, n_layers: int) -> list[nn.Module]:
    names = ft_config.module_fqns_per_model_fragment
    if not names:
        if ft_config.num_fragments <= 1:
            return [model]
        names = generate_llm_fqn_per_model_part(ft_config.num_fragments, n_layers, 1, 1)
    return module_split(model, names)
