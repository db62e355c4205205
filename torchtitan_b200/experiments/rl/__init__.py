"""Reinforcement-learning post-training (GRPO and relatives) on one node of B200s.

Roles, as in torchtitan/experiments/rl/unified: a :class:`Generator` that produces completions with
per-token log-probabilities, a :class:`Grader` that scores them, a :class:`PolicyTrainer` holding the
policy and a frozen reference model, and the :class:`RLTrainer` controller (generate -> score ->
group-mean advantages -> policy step -> weight sync). Instead of an external inference engine the
generator runs this framework's own model through a paged-KV engine (``engine.py``) using the same
kernels as training, which is what makes generator and trainer log-probabilities agree; roles live
in one process group (colocated on the same GPUs or on disjoint rank sets) and weights move through
a precomputed copy plan (``weight_sync.py``) instead of an RPC of full tensors.
"""

from .types import Episode

__all__ = ["Episode"]
