"""The rollout role: turns prompts into :class:`Episode` lists with this framework's own engine.

API and configuration names follow torchtitan/experiments/rl/unified/actors/generator.py:32-341
(``Generator`` is also exported as ``VLLMGenerator``): ``generate(prompt_texts, expected_answers)``
returns ``num_samples_per_prompt`` episodes per prompt carrying completion token ids and per-token
log-probabilities; ``update(version, state_dict)`` installs new policy weights. Differences by design:
the engine is ``engine.GenerationEngine`` (no external inference server), ``compile.cudagraph_mode``
other than ``none`` means the decode step is captured in CUDA graphs, and ``update`` also accepts the
trainer's flat bf16 arena (see ``weight_sync``). Generator data parallelism is by independent replicas;
a 0.6B-32B policy fits one 180 GB GPU, so the generator itself is not tensor-parallel.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

import torch

from torchtitan_b200.config import TORCH_DTYPE_MAP, ParallelismConfig
from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.tools.logging import logger

from .engine import GenerationEngine, PagedKVCache
from .types import Episode


@dataclass(kw_only=True, slots=True)
class GeneratorCompileConfig:
    backend: Literal["none", "eager", "inductor"] = "eager"
    """Kept for configuration compatibility; no tracing compiler is used here."""
    cudagraph_mode: Literal["none", "piecewise", "full", "full_and_piecewise"] = "piecewise"
    """Anything but ``none`` captures the batched decode step in CUDA graphs."""

    def __post_init__(self) -> None:
        if self.backend == "none" and self.cudagraph_mode in ("piecewise", "full_and_piecewise"):
            raise ValueError(
                f"cudagraph_mode='{self.cudagraph_mode}' requires piecewise graph capture which depends on "
                "torch.compile. Set backend to 'eager' or 'inductor'."
            )

    @property
    def is_eager(self) -> bool:
        return self.backend == "none" and self.cudagraph_mode == "none"


@dataclass(kw_only=True, slots=True)
class SamplingConfig:
    temperature: float = 0.8
    top_p: float = 0.95
    max_tokens: int = 100


class Generator(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        parallelism: ParallelismConfig = field(default_factory=ParallelismConfig)
        sampling: SamplingConfig = field(default_factory=SamplingConfig)
        attention_backend: str = "FLASH_ATTN"
        model_dtype: str = "bfloat16"
        gpu_memory_limit: float = 0.9
        compile: GeneratorCompileConfig = field(default_factory=GeneratorCompileConfig)
        num_samples_per_prompt: int = 8
        seed: int | None = None
        kv_block_size: int = 16
        max_kv_blocks: int | None = None
        """Cap on KV-cache blocks; by default ``gpu_memory_limit`` of the free memory is used."""

        def __post_init__(self):
            assert self.parallelism.data_parallel_shard_degree in (1, -1), (
                f"Generator does not support data parallel sharding, got dp_shard={self.parallelism.data_parallel_shard_degree}"
            )
            assert self.parallelism.data_parallel_replicate_degree == 1, (
                "Generator does not support data parallel replication, "
                f"got dp_replicate={self.parallelism.data_parallel_replicate_degree}"
            )

    def __init__(self, config: Config, *, model_spec, model_path: str = "", batch_invariant_mode: bool = False,
                 tokenizer=None, device: torch.device | str | None = None, model=None):
        self.config = config
        self.device = torch.device(device) if device is not None else torch.device(
            f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cpu")
        dtype = TORCH_DTYPE_MAP[config.model_dtype] if self.device.type == "cuda" else torch.float32
        if model is None:
            old = torch.get_default_dtype()
            torch.set_default_dtype(dtype)
            try:
                with torch.device("meta"):
                    model = model_spec.model.build()
            finally:
                torch.set_default_dtype(old)
            model.to_empty(device=self.device)
            with torch.no_grad():
                model.init_weights(buffer_device=self.device)
        for p in model.parameters():
            p.requires_grad_(False)
        self.model = model.eval()
        self.tokenizer = tokenizer
        self.policy_version = 0
        att = model.config.layer.attention
        n_kv, hd = (att.n_kv_heads or att.n_heads), (att.head_dim or model.config.dim // att.n_heads)
        per_block = PagedKVCache.bytes_per_block(len(model.layers), config.kv_block_size, n_kv, hd, dtype)
        if config.max_kv_blocks is not None:
            blocks = config.max_kv_blocks
        elif self.device.type == "cuda":
            free, total = torch.cuda.mem_get_info(self.device)
            budget = max(0, int(free - (1.0 - config.gpu_memory_limit) * total))
            blocks = max(256, min(budget // per_block, 1 << 20))
        else:
            blocks = 2048
        self.engine = GenerationEngine(
            self.model, block_size=config.kv_block_size, num_blocks=int(blocks),
            cudagraph=config.compile.cudagraph_mode != "none", eos_id=getattr(tokenizer, "eos_id", None),
        )
        self._rng = None
        if config.seed is not None:
            self._rng = torch.Generator(device=self.device)
            self._rng.manual_seed(config.seed)
        logger.info(f"Generator ready: {blocks} KV blocks of {config.kv_block_size} tokens, dtype {dtype}")

    # ---- weights ---------------------------------------------------------------------------------------
    def update(self, version: int, state_dict: dict | None = None) -> None:
        """Install policy weights (full tensors keyed like ``model.state_dict()``); captured decode graphs stay
        valid because parameters are overwritten in place."""
        if state_dict is not None:
            own = dict(self.model.named_parameters())
            own.update(dict(self.model.named_buffers()))
            with torch.no_grad():
                for k, v in state_dict.items():
                    if k in own and own[k].shape == v.shape:
                        own[k].copy_(v)
        self.policy_version = version
        arena = getattr(self, "arena", None)
        if arena is not None:
            self.engine.weight_half = arena.active

    # ---- rollouts --------------------------------------------------------------------------------------
    def generate(self, prompt_texts: list[str], expected_answers: list[str] | None = None) -> list[Episode]:
        tok = self.tokenizer
        assert tok is not None, "Generator.generate needs a tokenizer"
        prompts = [tok.encode(t, add_bos=True, add_eos=False) for t in prompt_texts]
        return self.generate_from_ids(prompts, expected_answers)

    def generate_from_ids(self, prompts: list[list[int]], expected_answers: list[str] | None = None) -> list[Episode]:
        sc = self.config.sampling
        n = self.config.num_samples_per_prompt
        seqs = self.engine.generate(prompts, n_samples=n, max_tokens=sc.max_tokens, temperature=sc.temperature,
                                    top_p=sc.top_p, generator=self._rng)
        eps = []
        for s in seqs:
            ids = s.tokens[:-1] if s.hit_eos else s.tokens
            text = self.tokenizer.decode(ids) if self.tokenizer is not None else ""
            eps.append(Episode(
                policy_version=self.policy_version, prompt_token_ids=list(prompts[s.prompt]), text=text, token_ids=list(s.tokens),
                token_log_probs=list(s.logprobs), expected_answer=(expected_answers[s.prompt] if expected_answers else ""),
                group_id=f"v{self.policy_version}-p{s.prompt}", finished=s.hit_eos,
            ))
        return eps


VLLMGenerator = Generator  # configuration-compatible name
