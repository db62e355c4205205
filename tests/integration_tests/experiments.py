"""One suite per experiment. Reference: torchtitan/experiments/{vlm,autoparallel,transformers_modeling_backend,ft,
graph_trainer}/tests/integration_tests.py (the same record type, one list builder per experiment)."""

from . import OverrideDefinitions as T

TP = "--parallelism.tensor_parallel_degree"
SHARD = "--parallelism.data_parallel_shard_degree"
PP = "--parallelism.pipeline_parallel_degree"


def build_vlm_test_list() -> list[T]:
    v = dict(module="vlm", config="vlm_debugmodel")
    return [T([[]], "VLM FSDP", "vlm_fsdp", ngpu=2, **v),
            T([[f"{SHARD} 2", "--parallelism.data_parallel_replicate_degree 2"]], "VLM HSDP", "vlm_hsdp", ngpu=4, **v)]


def build_autoparallel_test_list() -> list[T]:
    return [T([[]], "Planner-chosen layout, Llama", "autoparallel_llama3", ngpu=4, module="autoparallel",
              config="autoparallel_llama3_debugmodel"),
            T([[]], "Planner-chosen layout, DeepSeek V3", "autoparallel_deepseek_v3", ngpu=4, module="autoparallel",
              config="autoparallel_deepseek_v3_debugmodel")]


def build_transformers_backend_test_list() -> list[T]:
    # wrapped Hugging Face models take data-parallel layouts and tensor parallel; pipeline / context parallel over an
    # arbitrary Hugging Face module tree are not built here
    h = dict(module="transformers_modeling_backend", config="transformers_modeling_backend_debugmodel")
    return [T([[]], "Hugging Face model, FSDP", "hf_fsdp", ngpu=2, **h),
            T([[f"{SHARD} 2", "--parallelism.data_parallel_replicate_degree 2"]], "Hugging Face model, HSDP", "hf_hsdp", ngpu=4, **h),
            T([[f"{SHARD} 2", f"{TP} 2"]], "Hugging Face model, FSDP + TP", "hf_fsdp+tp", ngpu=4, **h),
            T([["--checkpoint.enable"], ["--checkpoint.enable", "--training.steps 20"]], "Hugging Face model, save and resume",
              "hf_checkpoint", ngpu=2, **h)]


def build_ft_test_list() -> list[T]:
    # the job is a 100-step DiLoCo run over NCCL replica groups: a short one on whatever backend the ranks have
    short = ["--training.steps 20", "--fault_tolerance.sync_steps 4", "--fault_tolerance.process_group gloo",
             "--comm.train_timeout_seconds 100", "--profiling.no-enable-profiling"]
    return [T([["--fault_tolerance.enable", "--fault_tolerance.replica_id 0", "--fault_tolerance.group_size 1", *short]],
              "Fault-tolerant trainer, one replica group, DiLoCo", "ft_single_group", ngpu=2, module="ft", config="llama3_ft_debugmodel"),
            T([["--fault_tolerance.enable", "--fault_tolerance.replica_id 0", "--fault_tolerance.group_size 1",
                "--fault_tolerance.semi_sync_method None", *short]],
              "Fault-tolerant trainer, one replica group, synchronous", "ft_single_group_sync", ngpu=2, module="ft",
              config="llama3_ft_debugmodel")]


def build_graph_trainer_test_list() -> list[T]:
    g = dict(module="graph_trainer")
    return [T([[]], "Graph trainer, Llama", "graph_llama3", ngpu=2, config="graph_trainer_llama3_debugmodel", **g),
            T([[f"{SHARD} 2", f"{TP} 2"]], "Graph trainer, Llama, FSDP + TP", "graph_llama3_fsdp+tp", ngpu=4,
              config="graph_trainer_llama3_debugmodel", **g),
            T([[]], "Graph trainer with CUDA-graph capture", "graph_llama3_cudagraph", ngpu=1, needs_gpu=True,
              config="graph_trainer_llama3_debugmodel_cudagraph", **g),
            T([["--parallelism.expert_parallel_degree 2"]], "Graph trainer, DeepSeek V3, FSDP + EP", "graph_deepseek_v3_ep", ngpu=4,
              config="graph_trainer_deepseek_v3_debugmodel", **g)]
