"""Context parallel under the reference's module name (torchtitan/distributed/context_parallel.py)."""

from torchtitan_b200.parallel.cp import (  # noqa: F401
    RingAttention,
    apply_cp_to_attention_module,
    cp_shard,
    prepare_context_parallel_input,
)

__all__ = ["RingAttention", "apply_cp_to_attention_module", "cp_shard", "prepare_context_parallel_input"]
