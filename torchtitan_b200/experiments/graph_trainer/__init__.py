"""Graph trainer: whole-step execution plans without a tracing compiler.

The reference experiment (torchtitan/experiments/graph_trainer) exports the joint forward/backward
graph and rewrites it with FX passes (collective bucketing and overlap scheduling, CUDA-graph
wrapping, graph-level activation checkpointing, reshard-after-forward annotation, extra process
group for all-gathers, optional Inductor lowering). On B200 the same ends are reached at run time:
the FSDP runtime already issues bucketed, prefetched collectives on side streams, so the named passes
become *plan edits* (how parameters are bucketed into units, prefetch depth, reshard policy, which ops
are saved) and ``cudagraph`` captures the forward+backward of a step into a CUDA graph that is
replayed with static input buffers. Passes that would hand the step to the Inductor compiler are
rejected with an explanation rather than silently ignored."""

from .configs import GraphTrainerCompileConfig, GraphTrainerConfig, to_graph_trainer_config
from .cudagraph import CUDAGraphWrapper
from .trainer import GraphTrainer

__all__ = ["GraphTrainer", "GraphTrainerConfig", "GraphTrainerCompileConfig", "to_graph_trainer_config", "CUDAGraphWrapper"]
