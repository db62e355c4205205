"""Extended fault-tolerance configuration (semi-sync knobs), fields as in
torchtitan/experiments/ft/config/job_config.py:13-80."""

from dataclasses import dataclass, field

from torchtitan_b200.experiments.ft.manager import FTManager


@dataclass(kw_only=True, slots=True)
class FaultTolerance(FTManager.Config):
    sync_steps: int = 5
    """Inner steps between synchronisations (LocalSGD / DiLoCo)."""
    should_quantize: bool = False
    """Quantise pseudo-gradients (bf16) before the cross-replica all-reduce."""
    fragment_sync_delay: int = 0
    """Steps a fragment's all-reduce may lag behind the point where it was prepared (streaming DiLoCo)."""
    fragment_update_alpha: float = 0.0
    """Mix of local and global parameters after a sync: 0 = take the global ones."""
    module_fqns_per_model_fragment: list[list[str]] = field(default_factory=list)
    """Explicit fragment split, one list of module names per fragment."""
    num_fragments: int = 1
    """Number of fragments when no explicit split is given (layers are divided evenly)."""
