from .model import BaseModel
from .model_converter import ModelConverter, ModelConvertersContainer
from .model_spec import FaultTolerantModelSpec, ModelSpec
from .module import Module
from .state_dict_adapter import BaseStateDictAdapter, StateDictAdapter

__all__ = [
    "BaseModel",
    "Module",
    "ModelSpec",
    "FaultTolerantModelSpec",
    "ModelConverter",
    "ModelConvertersContainer",
    "BaseStateDictAdapter",
    "StateDictAdapter",
]
