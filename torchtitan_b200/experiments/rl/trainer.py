"""The learning role: policy + frozen reference model, one optimizer step per batch of episodes.

Parity: torchtitan/experiments/rl/unified/actors/trainer.py:41-355 (configuration sections; episodes
sharded round-robin over data-parallel ranks; reference log-probabilities without grad; GRPO/PPO loss
with ``kl_coef=0.1``; generator-vs-trainer log-probability check; gradient averaging over DP; clipping;
metrics dict; ``get_weights`` returns full tensors). Differences by design: all of a rank's episodes are
packed into one document-masked row, so a step is one forward/backward; models are built through the
``ModelSpec`` and parallelised with the framework's own FSDP / tensor parallel.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import TORCH_DTYPE_MAP, ActivationCheckpointConfig, CommConfig, CompileConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.parallel import ParallelDims
from torchtitan_b200.parallel import utils as dist_utils
from torchtitan_b200.tools.logging import logger

from .losses import compute_policy_gradient_loss, compute_token_log_probs_packed, verify_logprob_identity
from .types import Episode
from .weight_sync import full_tensor


def _greedy_pack(lengths: list[int], cap: int) -> list[list[int]]:
    groups, cur, tok = [], [], 0
    for j, n in enumerate(lengths):
        if cur and tok + n > cap:
            groups.append(cur)
            cur, tok = [], 0
        cur.append(j)
        tok += n
    if cur:
        groups.append(cur)
    return groups


def plan_microbatches(lengths_by_rank: list[list[int]], rank: int, cap: int) -> tuple[list[list[int]], int]:
    """Micro-batches (lists of local episode indices) for ``rank`` such that every rank runs the same number of them.

    Each rank's episodes are packed greedily under ``cap`` tokens; a rank with fewer micro-batches than the largest count
    splits its biggest ones, and when it has no episode left to split it repeats its first micro-batch (the caller gives
    the repeats zero weight). Returns ``(groups, n_real)``: ``groups[n_real:]`` are the repeats."""
    target = max(len(_greedy_pack(l, cap)) for l in lengths_by_rank)
    groups = _greedy_pack(lengths_by_rank[rank], cap)
    if not groups:
        raise ValueError(f"data-parallel rank {rank} has no episode: need at least one episode per trainer rank")
    while len(groups) < target:
        k = max(range(len(groups)), key=lambda i: len(groups[i]))
        if len(groups[k]) < 2:
            break
        g = groups.pop(k)
        groups[k:k] = [g[: len(g) // 2], g[len(g) // 2:]]
    n_real = len(groups)
    return groups + [groups[0]] * (target - n_real), n_real


class PolicyTrainer(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        optimizer: OptimizersContainer.Config = field(default_factory=OptimizersContainer.Config)
        lr_scheduler: LRSchedulersContainer.Config = field(default_factory=LRSchedulersContainer.Config)
        training: TrainingConfig = field(default_factory=TrainingConfig)
        parallelism: ParallelismConfig = field(default_factory=ParallelismConfig)
        comm: CommConfig = field(default_factory=CommConfig)
        objective: str = "grpo"
        """``grpo`` (sequence-level ratio against the reference model, KL penalty) or ``dapo`` (token-level
        ratio against the generator's log-probabilities, asymmetric clipping, no KL)."""
        kl_coef: float = 0.1
        ppo_clip_eps: float = 0.2
        entropy_coef: float = 0.01
        clip_low: float = 0.2
        clip_high: float = 0.28
        max_tokens_per_microbatch: int = 16384
        """Episodes of a rank are packed into rows of at most this many tokens; gradients accumulate over the rows."""

    def __init__(self, config: Config, *, model_spec, batch_invariant_mode: bool = False, hf_assets_path: str = "",
                 device: torch.device | str | None = None, group=None, ranks: list[int] | None = None):
        self.config, self.model_spec = config, model_spec
        if device is None:
            device = f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.parallel_dims = self.make_parallel_dims(config, world, ranks)
        if getattr(self.parallel_dims, "_base", None) is not None:
            self.parallel_dims.build_mesh()              # collective with the non-trainer ranks (see make_parallel_dims)
        if world > 1 and self.device.type == "cuda":
            # one seed for the trainer ranks, agreed inside their own group: DTensor's default start-up sync is a
            # broadcast over the whole job, which the generator ranks never enter
            t = torch.tensor([torch.initial_seed() % 2**62], dtype=torch.int64, device=self.device)
            dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            dist_utils.seed_dtensor_rng(self.parallel_dims.world_mesh, int(t.item()))
        self.sd_adapter = model_spec.state_dict_adapter(model_spec.model, hf_assets_path) if model_spec.state_dict_adapter else None
        self.model = self._build_model(hf_assets_path, trainable=True)
        self.model_parts = [self.model]
        self.needs_ref = config.objective != "dapo" and config.kl_coef != 0.0
        self.ref_model = None
        if self.needs_ref or config.objective != "dapo":
            self.ref_model = self._build_model(hf_assets_path, trainable=False)
            self._copy_weights(self.model, self.ref_model)
        self.optimizers = config.optimizer.build(model_parts=self.model_parts)
        self.lr_schedulers = config.lr_scheduler.build(optimizers=self.optimizers, training_steps=config.training.steps)
        self.policy_version = 0
        pd = self.parallel_dims
        self.dp_size = pd.dp_replicate * pd.dp_shard
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.dp_rank = rank // pd.non_data_parallel_size
        self.dp_enabled = pd.dp_enabled
        # the packed row is fed to 128-token attention tiles on the GPU
        self._pad_to = 128 * max(1, pd.tp) if self.device.type == "cuda" else max(1, pd.tp)

    @staticmethod
    def make_parallel_dims(config: "PolicyTrainer.Config", world: int, ranks: list[int] | None = None) -> ParallelDims:
        """The trainer's dims over ``ranks`` of the job. When that is a strict subset, every other rank of the job must
        build the same object and call ``build_mesh()`` once (process-group creation is a collective of the whole job)."""
        p = config.parallelism
        pd = ParallelDims(
            dp_shard=p.data_parallel_shard_degree, dp_replicate=p.data_parallel_replicate_degree, cp=p.context_parallel_degree,
            tp=p.tensor_parallel_degree, pp=p.pipeline_parallel_degree, ep=p.expert_parallel_degree,
            etp=p.expert_tensor_parallel_degree, world_size=world,
        )
        if ranks is not None and dist.is_initialized() and len(ranks) != dist.get_world_size():
            pd.set_base_ranks(ranks)
        return pd

    # ---- construction -----------------------------------------------------------------------------------
    def _build_model(self, hf_assets_path: str, trainable: bool):
        cfg = self.config
        dtype = TORCH_DTYPE_MAP[cfg.training.dtype]
        old = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            with torch.device("meta"):
                model = self.model_spec.model.build()
        finally:
            torch.set_default_dtype(old)
        pd = self.parallel_dims
        managed = pd.world_size > 1 or self.device.type == "cuda"   # one GPU: bf16 compute over fp32 master shards
        if managed:
            # the policy loss reads per-token log-probabilities of arbitrary labels: it needs the whole vocabulary on
            # every rank, so the output projection gathers its tensor-parallel shards (no loss parallel)
            import dataclasses

            par = dataclasses.replace(cfg.parallelism, disable_loss_parallel=True) if pd.tp_enabled else cfg.parallelism
            model = self.model_spec.parallelize_fn(
                model, parallel_dims=pd, training=cfg.training, model_converters=None, parallelism=par,
                compile_config=CompileConfig(), ac_config=ActivationCheckpointConfig(mode="none"), dump_folder="",
            )
        model.to_empty(device=self.device)
        with torch.no_grad():
            model.init_weights(buffer_device=self.device)
        if managed:
            from torchtitan_b200.parallel import fsdp
            from torchtitan_b200.parallel.tp import finalize_tp

            fsdp.materialize(model)
            if pd.tp_enabled or pd.ep_enabled:
                finalize_tp(model)
        if hf_assets_path and self.sd_adapter is not None and os.path.isdir(hf_assets_path) and any(
                f.endswith(".safetensors") for f in os.listdir(hf_assets_path)):
            self._load_initial_hf_weights(model, hf_assets_path)
        if trainable:
            model.train()
        else:
            for q in model.parameters():
                q.requires_grad_(False)
            model.eval()
        return model

    def _load_initial_hf_weights(self, model, checkpoint_path: str) -> None:
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import StateDictOptions, set_model_state_dict

        reader = self.sd_adapter.get_hf_storage_reader(checkpoint_path)
        hf_sd = self.sd_adapter.to_hf(model.state_dict())
        dcp.load(hf_sd, storage_reader=reader)
        set_model_state_dict(model=model, model_state_dict=self.sd_adapter.from_hf(hf_sd), options=StateDictOptions(strict=True))
        logger.info(f"Loaded initial weights from {checkpoint_path}")

    @staticmethod
    @torch.no_grad()
    def _copy_weights(src, dst) -> None:
        d = dict(dst.named_parameters())
        for n, p in src.named_parameters():
            a = d[n].to_local() if hasattr(d[n], "to_local") else d[n]
            b = p.to_local() if hasattr(p, "to_local") else p
            a.copy_(b)

    # ---- endpoints ----------------------------------------------------------------------------------------
    def get_weights(self) -> dict:
        """Full (unsharded) tensors keyed like the model's state dict."""
        params = dict(self.model.named_parameters(remove_duplicate=False))   # the parameter objects carry the sharding tags
        return {k: full_tensor(params.get(k, v)) for k, v in self.model.state_dict().items() if torch.is_tensor(v)}

    def step(self, episodes: list[Episode]) -> dict:
        cfg = self.config
        advantages = torch.tensor([ep.advantage for ep in episodes])
        rewards = torch.tensor([ep.reward for ep in episodes])
        mine = list(range(self.dp_rank, len(episodes), self.dp_size))
        gen_ids = [episodes[i].token_ids for i in mine]
        prompt_ids = [episodes[i].prompt_token_ids for i in mine]
        gen_lps = [episodes[i].token_log_probs for i in mine]
        my_adv = advantages[mine]

        # micro-batches: greedy packing of this rank's episodes into rows of bounded length. Every forward/backward of a
        # sharded model is a collective of the data-parallel group, so all its ranks must run the SAME number of them:
        # each rank plans the packing of every rank (all hold the full episode list) and matches the largest count.
        lens = [[len(episodes[i].prompt_token_ids) + len(episodes[i].token_ids) for i in range(r, len(episodes), self.dp_size)]
                for r in range(self.dp_size)]
        groups, n_real = plan_microbatches(lens, self.dp_rank, cfg.max_tokens_per_microbatch)
        n_seqs, n_toks = len(mine), max(1, sum(len(g) for g in gen_ids))
        self.optimizers.zero_grad()
        loss_total, token_lps, agg = 0.0, [None] * len(mine), {}
        for gi, idx in enumerate(groups):
            real = gi < n_real       # the rest repeat a micro-batch with zero weight, only to keep the collectives paired
            sel = lambda xs: [xs[j] for j in idx]  # noqa: E731
            ref_lps = None
            if self.ref_model is not None and cfg.objective != "dapo":
                with torch.no_grad():
                    ref_lps = compute_token_log_probs_packed(self.ref_model, sel(prompt_ids), sel(gen_ids), self.device, self._pad_to)
            loss, m, lps = compute_policy_gradient_loss(
                self.model, sel(gen_ids), sel(prompt_ids), my_adv[idx], ref_lps, kl_coef=cfg.kl_coef,
                ppo_clip_eps=cfg.ppo_clip_eps, entropy_coef=cfg.entropy_coef, objective=cfg.objective,
                gen_token_log_probs=sel(gen_lps), clip_low=cfg.clip_low, clip_high=cfg.clip_high, pad_to=self._pad_to,
                n_seqs_total=n_seqs, n_tokens_total=n_toks,
            )
            # data-parallel mean of the per-rank losses: FSDP sums gradients, so scale by 1 / dp_size
            if not real:
                (loss * 0.0).backward()
                continue
            (loss / self.dp_size if self.dp_enabled else loss).backward()
            loss_total += loss.item()
            for j, t in zip(idx, lps):
                token_lps[j] = t.detach()
            for k, v in m.items():
                agg[k] = agg.get(k, 0.0) + (v if k in ("pg_loss", "entropy", "kl_div") else v * len(idx) / n_seqs)
        loss_metrics = agg
        loss = torch.tensor(loss_total)
        check = verify_logprob_identity(gen_lps, token_lps)
        if self.dp_enabled and not self._fsdp_owns_grads():
            for p in self.model.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=self.parallel_dims.get_mesh("batch").get_group()
                                    if self.parallel_dims.get_optional_mesh("batch") is not None else None)
        grad_norm = dist_utils.clip_grad_norm_(
            [p for m in self.model_parts for p in m.parameters()], cfg.training.max_norm, foreach=True,
            pp_mesh=self.parallel_dims.get_optional_mesh("pp"),
        )
        self.optimizers.step()
        self.lr_schedulers.step()
        self.policy_version += 1
        return {
            "loss": loss.item(), "reward_mean": rewards.mean().item(),
            "reward_std": rewards.std().item() if len(rewards) > 1 else 0.0,
            "advantage_mean": advantages.mean().item(), "advantage_std": advantages.std().item() if len(advantages) > 1 else 0.0,
            "sample_completion": episodes[0].text[:80], "policy_version": self.policy_version,
            "grad_norm": float(grad_norm), "logprob_diff_mean": check["logprob_diff_mean"],
            "logprob_diff_max": check["logprob_diff_max"], "logprob_max_delta": check["logprob_max_delta"],
            "logprob_bitwise_identical": check["logprob_bitwise_identical"], **loss_metrics,
        }

    def _fsdp_owns_grads(self) -> bool:
        from torchtitan_b200.parallel import fsdp

        return bool(fsdp.fsdp_units(self.model))
