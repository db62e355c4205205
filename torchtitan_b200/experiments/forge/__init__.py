"""``ForgeEngine``: everything the trainer builds (meshes, parallelised model parts, loss, optimizers, schedulers,
checkpointer, contexts) without a training loop, for post-training stacks that drive the steps themselves.
Parity: torchtitan/experiments/forge/engine.py:35-298 and example_train.py:35-469."""

from .engine import ForgeEngine

__all__ = ["ForgeEngine"]
