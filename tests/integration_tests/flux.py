"""FLUX suite. Reference: tests/integration_tests/flux.py:23-140."""

from . import OverrideDefinitions as T


def build_flux_test_list() -> list[T]:
    fx = dict(module="flux", config="flux_debugmodel")
    return [
        T([[]], "FLUX FSDP", "flux_fsdp", ngpu=2, **fx),
        T([["--parallelism.data_parallel_shard_degree 2", "--parallelism.data_parallel_replicate_degree 2"]], "FLUX HSDP",
          "flux_hsdp", ngpu=4, **fx),
        T([["--parallelism.data_parallel_shard_degree 2", "--parallelism.context_parallel_degree 2"]], "FLUX FSDP + CP",
          "flux_fsdp+cp", ngpu=4, **fx),
        T([["--validator.enable"]], "FLUX with validation images", "flux_validation", ngpu=2, **fx),
        T([["--checkpoint.enable"], ["--checkpoint.enable", "--training.steps 20"]], "FLUX save and resume", "flux_checkpoint",
          ngpu=2, **fx),
        # train with validation and save, then generate images for the prompt file from that checkpoint
        T([["--parallelism.data_parallel_shard_degree 2", "--parallelism.data_parallel_replicate_degree 2",
            "--parallelism.context_parallel_degree 2", "--validator.enable", "--validator.steps 5", "--checkpoint.enable"],
           ["--parallelism.data_parallel_shard_degree 2", "--parallelism.data_parallel_replicate_degree 2",
            "--parallelism.context_parallel_degree 2", "--checkpoint.enable",
            "--checkpoint.exclude_from_loading lr_scheduler,dataloader,optimizer"]],
          "HSDP+CP+Validation+Inference", "hsdp+cp+validation+inference", ngpu=8,
          env=({}, {"TRAIN_FILE": "torchtitan_b200.models.flux.inference.infer"}), **fx),
    ]
