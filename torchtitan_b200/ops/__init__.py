"""Hot ops. On a CUDA device each op launches this framework's sm_100a kernel (and raises if
the native library is not built); on CPU it runs the PyTorch definition in ``reference``.
"""

from . import reference
from .functional import (
    attention,
    cross_entropy_sum,
    linear,
    native_available,
    rms_norm,
    rope,
    swiglu,
    token_logprobs,
)

__all__ = [
    "reference",
    "linear",
    "rms_norm",
    "rope",
    "swiglu",
    "attention",
    "cross_entropy_sum",
    "token_logprobs",
    "native_available",
]
