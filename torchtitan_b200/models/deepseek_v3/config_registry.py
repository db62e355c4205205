"""DeepSeek-V3 job configurations (names as in torchtitan/models/deepseek_v3/config_registry.py:28-135)."""

from torchtitan_b200.components.quantization.float8 import Float8GroupedMMConverter, Float8LinearConverter
from torchtitan_b200.models import job_configs as _jobs
from torchtitan_b200.trainer import Trainer

from . import model_registry

_COSINE = dict(decay_ratio=0.8, decay_type="cosine", min_lr_factor=0.1)


def _experts(ep: int, **more) -> dict:
    return dict(expert_parallel_degree=ep, expert_tensor_parallel_degree=1, **more)


def deepseek_v3_debugmodel() -> Trainer.Config:
    return _jobs.debug_job(model_registry("debugmodel"), ac=("selective", "op"), parallel=_experts(1))


def deepseek_v3_debugmodel_flex_attn() -> Trainer.Config:
    return _jobs.debug_job(model_registry("debugmodel_flex_attn"), ac=("selective", "op"), parallel=_experts(1))


def deepseek_v3_16b() -> Trainer.Config:
    return _jobs.text_job(model_registry("16B"), assets="./assets/hf/deepseek-moe-16b-base", dataset="c4", lr=2.2e-4, batch=4, seq=4096,
                    steps=1000, schedule=_COSINE, checkpoint=dict(interval=10), compile=dict(enable=True, components=["loss"]),
                    parallel=_experts(8, pipeline_parallel_schedule="Interleaved1F1B"))


def deepseek_v3_671b() -> Trainer.Config:
    return _jobs.text_job(model_registry("671B"), assets="./assets/hf/DeepSeek-V3.1-Base", dataset="c4", lr=2.2e-4, batch=4, seq=4096,
                    steps=10000, schedule=dict(warmup_steps=2000, **_COSINE), checkpoint=dict(interval=500),
                    compile=dict(enable=True, components=["loss"]),
                    parallel=_experts(1, pipeline_parallel_schedule="Interleaved1F1B"),
                    converters=[Float8LinearConverter.Config(filter_fqns=["output", "router.gate"]),
                                Float8GroupedMMConverter.Config(fqns=["experts"])])
