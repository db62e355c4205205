"""torchtitan_b200: a Blackwell (sm_100a) native LLM training and RL framework.

The package keeps the public surface of torchtitan 0.2.2 (``Trainer``, the
``--module/--config`` registry, ``ModelSpec``, DCP checkpoints) while the hot
path is hand-written CUDA for B200: tcgen05/TMEM GEMM and attention kernels,
TMA data movement, and collectives that read and write NVLink peer memory
directly from the kernels.
"""

__version__ = "0.1.0"
