"""``Linear``: an ``nn.Linear`` (same parameter names and state dict) whose forward runs the
framework GEMM. Parity: torchtitan/models/common/linear.py:14-56 (late-bound in/out
features, truncated-normal init with a per-call ``init_std`` override, zero bias)."""

from dataclasses import dataclass, field

import torch
import torch.nn as nn

import os

from torchtitan_b200 import ops
from torchtitan_b200.ops.wgrad_store import WeightGradStore
from torchtitan_b200.protocols.module import Module


# residual additions inside the output projections' GEMM epilogues (``Linear.add_to``); TT_RESIDUAL_EPILOGUE=0 adds afterwards
RESIDUAL_EPILOGUE = os.environ.get("TT_RESIDUAL_EPILOGUE", "1") == "1"


# input gradients of linears that share their input summed in GEMM epilogues (``project_together``); TT_FUSED_DGRAD=0: by autograd
FUSED_DGRAD = os.environ.get("TT_FUSED_DGRAD", "1") == "1"


class Linear(nn.Linear, Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        in_features: int = field(init=False)
        out_features: int = field(init=False)
        bias: bool = False
        init_mean: float = 0.0
        init_std: float = 0.02

    def __init__(self, config: Config):
        if not (hasattr(config, "in_features") and hasattr(config, "out_features")):
            raise TypeError(
                "Linear.Config requires 'in_features' and 'out_features' to be set "
                "(use Config.build(in_features=..., out_features=...))."
            )
        super().__init__(config.in_features, config.out_features, bias=config.bias)
        self._init_mean, self._init_std = config.init_mean, config.init_std
        self.quant = None  # a QuantRecipe once a quantisation converter selected this layer

    def forward(self, x):
        if self.quant is not None:
            from torchtitan_b200.ops.quant import quant_linear

            return quant_linear(x, self.weight, self.bias, self.quant)
        return ops.linear(x, self.weight, self.bias)

    def add_to(self, residual, x):
        """``residual + self(x)``. On CUDA in bf16 the addition runs in the epilogue of the GEMM (one kernel, no extra pass
        over the output); a layer that is quantised, has a bias or had its forward replaced (tensor parallel) adds after
        the call."""
        if RESIDUAL_EPILOGUE and self.quant is None and self.bias is None and "forward" not in self.__dict__ and x.is_cuda \
                and not WeightGradStore.enabled:
            from torchtitan_b200.ops import cuda_ops

            y = cuda_ops.linear_residual(x, self.weight, residual)
            if y is not None:
                return y
        return residual + self(x)

    def init_weights(self, **kwargs) -> None:
        std = kwargs.get("init_std")
        nn.init.trunc_normal_(self.weight, mean=self._init_mean, std=self._init_std if std is None else std)
        if self.bias is not None:
            nn.init.zeros_(self.bias)


def with_residual(module, residual, *args):
    """``residual + module(*args)``. A module whose forward takes ``residual`` adds it in its output projection; one
    whose forward was replaced (tensor parallel gathers / scatters around it) gets the addition after the call, where
    the shapes match again."""
    if "forward" in module.__dict__:
        return residual + module(*args)
    return module(*args, residual=residual)



def project_together(x, *linears):
    """``[lin(x) for lin in linears]``. Plain bf16 layers on CUDA run through one autograd node whose backward sums the
    input gradients inside the GEMMs; anything else (quantised, biased, tensor-parallel wrapped) is called one by one."""
    if FUSED_DGRAD and x.is_cuda and not WeightGradStore.enabled and torch.is_grad_enabled() and all(
            type(lin) is Linear and lin.quant is None and lin.bias is None and "forward" not in lin.__dict__ for lin in linears):
        from torchtitan_b200.ops import cuda_ops

        ys = cuda_ops.multi_linear(x, [lin.weight for lin in linears])
        if ys is not None:
            return ys
    return tuple(lin(x) for lin in linears)
