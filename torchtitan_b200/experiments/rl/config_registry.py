"""RL job configurations (names as in torchtitan/experiments/rl/unified/config_registry.py:28-140)."""

from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ParallelismConfig, TrainingConfig
from torchtitan_b200.models.qwen3 import model_registry

from .generator import Generator, GeneratorCompileConfig, SamplingConfig
from .simple_grpo_sum_digits import RLTrainer
from .trainer import PolicyTrainer


def _cfg(flavor: str, assets: str, *, lr: float, train_tp: int, gen_tp: int, samples: int, temp: float, max_tokens: int,
         steps: int, invariant: bool) -> RLTrainer.Config:
    return RLTrainer.Config(
        model_spec=model_registry(flavor), hf_assets_path=assets, num_steps=steps, batch_invariant_mode=invariant,
        trainer=PolicyTrainer.Config(
            optimizer=OptimizersContainer.Config(lr=lr),
            lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_type="linear"),
            training=TrainingConfig(),
            parallelism=ParallelismConfig(tensor_parallel_degree=train_tp, data_parallel_replicate_degree=1),
        ),
        generator=Generator.Config(
            model_dtype="bfloat16",
            compile=GeneratorCompileConfig(backend="eager", cudagraph_mode="piecewise"),
            # one 180 GB GPU holds these policies: generator ranks are independent replicas, not a TP group
            parallelism=ParallelismConfig(tensor_parallel_degree=1, data_parallel_replicate_degree=1),
            num_samples_per_prompt=samples,
            sampling=SamplingConfig(temperature=temp, top_p=0.95, max_tokens=max_tokens),
            attention_backend="FLASH_ATTN",
        ),
    )


def rl_grpo_qwen3_0_6b() -> RLTrainer.Config:
    """Qwen3-0.6B: 2 trainer GPUs (TP 2) + generator replicas on the remaining ranks."""
    return _cfg("0.6B", "torchtitan_b200/experiments/rl/example_checkpoint/Qwen3-0.6B", lr=2e-6, train_tp=2, gen_tp=2, samples=8,
                temp=0.8, max_tokens=100, steps=10, invariant=True)


def rl_grpo_qwen3_1_7b() -> RLTrainer.Config:
    """Qwen3-1.7B: 2 trainer GPUs (TP 2) + 4 generator replicas."""
    return _cfg("1.7B", "torchtitan_b200/experiments/rl/example_checkpoint/Qwen3-1.7B", lr=2e-6, train_tp=2, gen_tp=4, samples=8,
                temp=0.8, max_tokens=100, steps=10, invariant=True)


def rl_grpo_qwen3_debug() -> RLTrainer.Config:
    """Small model, few steps; runs colocated on one GPU (or CPU) or as 1 trainer + 1 generator rank."""
    return _cfg("debugmodel", "./tests/assets/tokenizer", lr=8e-4, train_tp=1, gen_tp=1, samples=4, temp=1.0, max_tokens=50,
                steps=5, invariant=False)
