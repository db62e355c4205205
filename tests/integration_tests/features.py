"""Feature suite: one case per framework feature on the debug Llama model.

Reference: tests/integration_tests/features.py:23-560 (the same feature coverage; ``--compile.enable`` cases are
replaced by their eager forms since this framework has no tracing compiler)."""

from . import OverrideDefinitions as T

PP = "--parallelism.pipeline_parallel_degree"
SCHED = "--parallelism.pipeline_parallel_schedule"
TP = "--parallelism.tensor_parallel_degree"
CP = "--parallelism.context_parallel_degree"
SHARD = "--parallelism.data_parallel_shard_degree"
REPL = "--parallelism.data_parallel_replicate_degree"
CKPT = "--checkpoint.enable"


def build_features_test_list() -> list[T]:
    return [
        T([["--profiling.enable_profiling", "--metrics.enable_tensorboard"]], "default", "default"),
        T([["--activation_checkpoint.mode selective", "--activation_checkpoint.selective_ac_option op"]],
          "1D with per-op selective AC", "1d_sac_op"),
        T([["--activation_checkpoint.mode full"]], "1D with full AC", "1d_full_ac"),
        T([["--activation_checkpoint.mode memory_budget", "--activation_checkpoint.memory_budget 0.5"]],
          "1D with a memory budget", "1d_memory_budget"),
        T([[f"{TP} 2"]], "2D eager", "2d_eager"),
        T([[f"{TP} 2", "--parallelism.enable_async_tensor_parallel"]], "2D with fused async TP", "2d_asynctp", needs_gpu=True),
        T([[CKPT], [CKPT, "--training.steps 20"]], "Checkpoint: save, then load the full checkpoint and continue", "full_checkpoint"),
        T([[CKPT, "--checkpoint.folder hf_checkpoint", "--checkpoint.last_save_model_only", "--checkpoint.last_save_in_hf"],
           [CKPT, "--checkpoint.initial_load_path {dump}/hf_checkpoint/step-10", "--checkpoint.initial_load_model_only",
            "--checkpoint.initial_load_in_hf"]],
          "Checkpoint: model-only save and load in the Hugging Face definition and format", "model_only_hf_checkpoint"),
        T([[CKPT, "--checkpoint.folder hf_checkpoint", "--checkpoint.last_save_model_only", "--checkpoint.last_save_in_hf", f"{TP} 2"],
           [CKPT, "--checkpoint.initial_load_path {dump}/hf_checkpoint/step-10", "--checkpoint.initial_load_model_only",
            "--checkpoint.initial_load_in_hf"]],
          "Checkpoint: Hugging Face export written under TP, loaded under plain FSDP", "hf_checkpoint_across_layouts"),
        T([[CKPT, "--checkpoint.last_save_model_only"]], "Checkpoint: model-only save in fp32", "last_save_model_only_fp32"),
        T([[CKPT, "--checkpoint.last_save_model_only", "--checkpoint.export_dtype bfloat16"]],
          "Checkpoint: model-only save in bf16", "last_save_model_only_bf16"),
        T([[CKPT, "--checkpoint.async_mode async_with_pinned_mem"]], "Checkpoint: asynchronous save from pinned memory",
          "async_checkpoint", ngpu=2),
        T([["--training.enable_cpu_offload"]], "FSDP with shards, gradients and optimizer state in host memory", "fsdp_cpu_offload",
          ngpu=2),
        T([[f"{PP} 4", f"{SCHED} InterleavedZeroBubble"]], "PP looped zero bubble", "pp_looped_zero_bubble", ngpu=4),
        T([[f"{PP} 2", f"{SCHED} ZBVZeroBubble"]], "PP zero bubble (V-shaped)", "pp_zbv", ngpu=2),
        T([[f"{PP} 2", f"{SCHED} DualPipeV"]], "PP DualPipeV placement", "pp_dualpipev", ngpu=2),
        T([[f"{PP} 2", f"{SCHED} 1F1B", f"{SHARD} 1"]], "PP 1D 1F1B", "pp_1f1b", ngpu=2),
        T([[f"{PP} 2", f"{SCHED} GPipe", f"{SHARD} 1"]], "PP 1D GPipe", "pp_gpipe", ngpu=2),
        T([[f"{PP} 2", f"{SCHED} 1F1B", f"{SHARD} 2"],
           [f"{PP} 2", f"{SCHED} 1F1B", "--parallelism.pipeline_parallel_layers_per_stage 4", f"{SHARD} 2"]],
          "PP + DP 1F1B", "pp_dp_1f1b"),
        T([[f"{PP} 2", f"{SCHED} GPipe", f"{SHARD} 2"]], "PP + DP GPipe", "pp_dp_gpipe"),
        T([[f"{PP} 2", f"{TP} 2"]], "PP + TP", "pp_tp"),
        T([[CKPT, f"{PP} 2", f"{SHARD} 2", f"{TP} 2"], ["--training.steps 20", CKPT, f"{PP} 2", f"{SHARD} 2", f"{TP} 2"]],
          "PP + DP + TP with save and resume", "pp_dp_tp", ngpu=8),
        T([[f"{PP} 4", f"{SCHED} Interleaved1F1B"],
           [f"{PP} 4", f"{SCHED} Interleaved1F1B", "--parallelism.pipeline_parallel_layers_per_stage 1"]],
          "PP looped 1F1B", "pp_looped_1f1b", ngpu=4),
        T([[f"{PP} 2", f"{SCHED} PipelineScheduleMulti",
            "--parallelism.pipeline_parallel_schedule_csv ./tests/assets/custom_schedule.csv",
            "--training.local_batch_size 8"]],        # the file is written for 8 micro-batches
          "PP with a schedule read from a CSV file", "pp_custom_csv", ngpu=2),
        T([["--optimizer.name AdamW", "--optimizer.implementation foreach"]], "Foreach optimizer", "optimizer_foreach", ngpu=2),
        T([[f"{SHARD} 1", f"{REPL} 4"]], "DDP", "ddp", ngpu=4),
        T([[f"{SHARD} 2", f"{REPL} 2"]], "HSDP", "hsdp", ngpu=4),
        T([[f"{CP} 4", "--parallelism.context_parallel_rotate_method allgather"]], "CP (allgather)", "cp_allgather", ngpu=4),
        T([[f"{CP} 4", "--parallelism.context_parallel_rotate_method alltoall"]], "CP (alltoall)", "cp_alltoall", ngpu=4),
        T([[f"{CP} 2"]], "CP with document masks", "cp_document_masks", ngpu=2, config="llama3_debugmodel_flex_attn"),
        T([[f"{PP} 2", f"{SCHED} 1F1B"]], "PP with document masks", "pp_document_masks", ngpu=2, config="llama3_debugmodel_flex_attn"),
        T([[f"{PP} 2", f"{SCHED} Interleaved1F1B"]], "PP with packed-document attention", "pp_varlen", ngpu=2,
          config="llama3_debugmodel_varlen_attn"),
        T([[f"{SHARD} 2", f"{REPL} 2", f"{TP} 2"]], "HSDP + TP", "hsdp+tp", ngpu=8),
        T([[f"{SHARD} 2", f"{CP} 2"]], "FSDP + CP", "fsdp+cp", ngpu=4),
        T([[f"{SHARD} 1", f"{REPL} 2", f"{CP} 2"]], "HSDP + CP (without dp_shard)", "hsdp+cp_without_dp_shard", ngpu=4),
        T([[f"{SHARD} 2", f"{REPL} 2", f"{CP} 2"]], "HSDP + CP (with dp_shard)", "hsdp+cp_with_dp_shard", ngpu=8),
        T([[f"{SHARD} 2", f"{TP} 2", f"{CP} 2"]], "FSDP + TP + CP", "fsdp+tp+cp", ngpu=8),
        T([["--parallelism.fsdp_reshard_after_forward always"]], "Reshard after every forward", "fsdp_reshard_always", ngpu=2),
        T([[CKPT, "--training.steps 10"],
           [CKPT, "--checkpoint.exclude_from_loading lr_scheduler,dataloader,optimizer", f"{TP} 2", "--training.steps 20"]],
          "Checkpoint: load with some states left out, on another layout", "optional_checkpoint"),
        T([["--training.local_batch_size 8", "--training.global_batch_size 32"]], "Gradient accumulation",
          "gradient_accumulation", ngpu=2),
        T([["--validator.enable", "--validator.dataloader.dataset c4_test", f"{TP} 2", f"{CP} 2", f"{PP} 2",
            f"{SCHED} Interleaved1F1B"]], "Validation with TP, CP and PP", "validation_tp_cp_pp", ngpu=8),
        T([["--dataloader.num_workers 2", "--dataloader.pin_memory", "--dataloader.persistent_workers",
            "--dataloader.prefetch_factor 4"]], "Dataloader options from the command line", "dataloader_kwargs", ngpu=2),
        T([["--debug.deterministic", "--debug.seed 42"]], "Deterministic run with a fixed seed", "deterministic", ngpu=2),
        T([[]], "Optimizer step inside backward", "optimizer_in_backward", ngpu=2, config="llama3_debugmodel_opt_in_bwd"),
        T([[]], "Variable-length attention (document masks)", "varlen_attn", ngpu=2, config="llama3_debugmodel_varlen_attn"),
        T([[]], "Flex-style attention (document masks)", "flex_attn", ngpu=2, config="llama3_debugmodel_flex_attn"),
        T([[]], "float8 rowwise training", "float8", ngpu=2, config="llama3_debugmodel_float8", needs_gpu=True),
        T([[]], "float8 emulated on any device", "float8_emulate", ngpu=2, config="llama3_debugmodel_float8_emulate"),
    ]
