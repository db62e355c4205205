"""``ModelSpec``: everything the Trainer needs to know about one model flavor.

Parity: torchtitan/protocols/model_spec.py:28-51.
"""

import copy
from collections.abc import Callable
from dataclasses import dataclass
from typing import Any

import torch.nn as nn

from .model import BaseModel
from .state_dict_adapter import BaseStateDictAdapter

ParallelizeFunction = Callable[..., nn.Module]
PipeliningFunction = Callable[..., tuple]
LossFunctionBuilder = Callable[..., Callable]
PostOptimizerBuildFn = Callable[..., None]


@dataclass
class ModelSpec:
    name: str
    flavor: str
    model: BaseModel.Config
    parallelize_fn: ParallelizeFunction
    pipelining_fn: PipeliningFunction | None
    build_loss_fn: LossFunctionBuilder
    post_optimizer_build_fn: PostOptimizerBuildFn | None = None
    state_dict_adapter: type[BaseStateDictAdapter] | None = None

    def __post_init__(self):
        # a specification owns its model configuration: the trainer adapts it to the job (sequence length, vocabulary
        # size ...), which must not change the flavor registered for everybody else in the process
        self.model = copy.deepcopy(self.model)


@dataclass
class FaultTolerantModelSpec(ModelSpec):
    fragment_fn: Callable[..., Any] | None = None
