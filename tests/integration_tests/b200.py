"""GPU-only suite: the paths that exist only on a B200 (quantised GEMMs, fused compute + collective kernels, peer-memory
FSDP transport). Reference: tests/integration_tests/h100.py:14-80 (the float8 / async-TP cases that need recent GPUs)."""

from . import OverrideDefinitions as T

TP = "--parallelism.tensor_parallel_degree"
SHARD = "--parallelism.data_parallel_shard_degree"


def build_b200_tests_list() -> list[T]:
    return [
        T([[f"{TP} 2", "--parallelism.enable_async_tensor_parallel"]], "Fused all-gather/GEMM and GEMM/reduce-scatter under TP",
          "asynctp", ngpu=2, needs_gpu=True),
        T([[f"{SHARD} 2", f"{TP} 2", "--parallelism.enable_async_tensor_parallel"]], "FSDP + fused async TP", "fsdp+asynctp",
          ngpu=4, needs_gpu=True),
        T([[]], "float8 rowwise with float8 all-gather", "float8_fsdp", ngpu=2, needs_gpu=True, config="llama3_debugmodel_float8"),
        T([[f"{TP} 2"]], "float8 rowwise with TP", "float8_tp", ngpu=4, needs_gpu=True, config="llama3_debugmodel_float8"),
        T([["--parallelism.fsdp_reshard_after_forward never"]], "Peer-memory FSDP transport, parameters kept gathered",
          "fsdp_nvlink_no_reshard", ngpu=2, needs_gpu=True),
        T([["--activation_checkpoint.mode selective", "--activation_checkpoint.selective_ac_option op",
            "--activation_checkpoint.per_op_sac_mm_policy auto"]], "Per-op SAC with the memory-driven matmul policy",
          "sac_mm_auto", ngpu=2, needs_gpu=True),
    ]
