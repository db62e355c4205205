"""The reference's ``torchtitan.distributed`` module layout, for code written against it.

This framework keeps its parallelism runtime in ``torchtitan_b200.parallel`` (own FSDP runtime, tensor / context /
expert / pipeline parallel, peer-memory collectives). The modules of this package carry the reference's file names
(torchtitan/distributed/{parallel_dims,utils,activation_checkpoint,context_parallel,expert_parallel,pipeline_parallel,
tensor_parallel,fsdp}.py) and re-export the corresponding entry points, so ``from torchtitan_b200.distributed import
ParallelDims`` or ``from torchtitan_b200.distributed.utils import set_determinism`` work as they do there."""

import sys

from torchtitan_b200.parallel import parallel_dims, utils
from torchtitan_b200.parallel.parallel_dims import ParallelDims

# ``parallel_dims`` and ``utils`` correspond one to one: the same module objects under both names, so that patching an
# attribute through either path reaches the code that uses it.
sys.modules[__name__ + ".parallel_dims"] = parallel_dims
sys.modules[__name__ + ".utils"] = utils

__all__ = ["ParallelDims", "parallel_dims", "utils"]
