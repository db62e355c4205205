"""Model suite: every model family's debug configuration under the parallelisms it supports.

Reference: tests/integration_tests/models.py:14-160."""

from . import OverrideDefinitions as T

PP = "--parallelism.pipeline_parallel_degree"
SCHED = "--parallelism.pipeline_parallel_schedule"
TP = "--parallelism.tensor_parallel_degree"
CP = "--parallelism.context_parallel_degree"
SHARD = "--parallelism.data_parallel_shard_degree"
EP = "--parallelism.expert_parallel_degree"
ETP = "--parallelism.expert_tensor_parallel_degree"


def build_model_tests_list() -> list[T]:
    ds = dict(module="deepseek_v3", config="deepseek_v3_debugmodel")
    qw = dict(module="qwen3", config="qwen3_debugmodel")
    qm = dict(module="qwen3", config="qwen3_moe_debug")
    l4 = dict(module="llama4", config="llama4_debugmodel")
    go = dict(module="gpt_oss", config="gpt_oss_debugmodel")
    return [
        T([[f"{SHARD} 4", f"{EP} 2"]], "DeepSeek V3 FSDP + EP", "deepseek_v3_fsdp+ep", ngpu=4, **ds),
        T([[f"{SHARD} 4", f"{TP} 2", f"{EP} 4", f"{ETP} 1"]], "DeepSeek V3 FSDP + TP + EP", "deepseek_v3_fsdp+tp+ep", ngpu=8, **ds),
        T([[f"{SHARD} 2", f"{TP} 2", f"{EP} 2", f"{ETP} 2"]], "DeepSeek V3 FSDP + TP + EP + ETP", "deepseek_v3_fsdp+tp+ep+etp",
          ngpu=4, **ds),
        T([[f"{PP} 2", f"{SCHED} Interleaved1F1B", f"{SHARD} 2", f"{EP} 2"]], "DeepSeek V3 PP + FSDP + EP",
          "deepseek_v3_pp+fsdp+ep", ngpu=4, **ds),
        T([[f"{PP} 2", f"{SCHED} DualPipeV", f"{SHARD} 2", f"{EP} 2", "--training.local_batch_size 8"]],
          "DeepSeek V3 DualPipeV (forward / backward slots overlapping the expert exchanges) + FSDP + EP",
          "deepseek_v3_dualpipev+fsdp+ep", ngpu=4, **ds),
        T([[f"{SHARD} 2", f"{CP} 2"]], "DeepSeek V3 FSDP + CP", "deepseek_v3_fsdp+cp", ngpu=4, **ds),
        T([[]], "DeepSeek V3 with document masks", "deepseek_v3_flex", ngpu=2, module="deepseek_v3",
          config="deepseek_v3_debugmodel_flex_attn"),
        T([[f"{SHARD} 2", f"{TP} 2"]], "Qwen3 FSDP + TP", "qwen3_fsdp+tp", ngpu=4, **qw),
        T([[f"{SHARD} 2", f"{CP} 2"]], "Qwen3 FSDP + CP", "qwen3_fsdp+cp", ngpu=4, **qw),   # tied weights: no PP for this flavor
        T([[f"{SHARD} 4", f"{EP} 2"]], "Qwen3 MoE FSDP + EP", "qwen3_moe_fsdp+ep", ngpu=4, **qm),
        T([[f"{SHARD} 2", f"{TP} 2", f"{EP} 2", f"{ETP} 1"]], "Qwen3 MoE FSDP + TP + EP", "qwen3_moe_fsdp+tp+ep", ngpu=4, **qm),
        T([[f"{SHARD} 2", f"{EP} 2", "--parallelism.expert_parallel_comm_backend deepep"]],
          "Qwen3 MoE with the peer-memory dispatcher", "qwen3_moe_nvlink_ep", ngpu=2, needs_gpu=True, **qm),
        T([[f"{SHARD} 4", f"{EP} 2"]], "Llama 4 FSDP + EP", "llama4_fsdp+ep", ngpu=4, **l4),
        T([[f"{PP} 2", f"{SHARD} 2", f"{TP} 2"]], "Llama 4 PP + FSDP + TP", "llama4_pp+fsdp+tp", ngpu=8, **l4),
        T([[f"{SHARD} 4", f"{EP} 2"]], "GPT-OSS FSDP + EP", "gpt_oss_fsdp+ep", ngpu=4, **go),
        T([[f"{SHARD} 2", f"{TP} 2", f"{EP} 2", f"{ETP} 1"]], "GPT-OSS FSDP + TP + EP", "gpt_oss_fsdp+tp+ep", ngpu=4, **go),
    ]
