"""GRPO on the sum-of-digits task: the RL controller.

``RLTrainer`` follows torchtitan/experiments/rl/unified/simple_grpo_sum_digits.py:105-387: evaluate,
then per step create ``num_episodes_per_step`` questions, generate ``num_samples_per_prompt``
completions each, score, subtract the group mean reward, take one policy step, sync weights to the
generator, log; evaluate again at the end. Roles run in this process (one process per GPU):

* 1 rank: trainer and generator are colocated on the same GPU and the generator's weights are refreshed
  by an on-device cast/copy into its parameter arena;
* several ranks: the first ``trainer world size`` ranks train, the remaining ranks are generator
  replicas (prompts are split between them); weights move with one arena broadcast, episodes with
  object collectives.

``async_mode`` (one step off-policy): generation for step ``t + 1`` is issued with the weights of step
``t - 1`` while the trainer works on step ``t``; on separate rank sets the two overlap fully.

Run: ``python -m torchtitan_b200.experiments.rl.simple_grpo_sum_digits --module rl --config rl_grpo_qwen3_debug``.
"""

from __future__ import annotations

import re
import time
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.protocols.model_spec import ModelSpec
from torchtitan_b200.tools.logging import init_logger, logger

from .generator import Generator
from .grader import Grader, group_mean_advantages
from .sum_digits import SumDigitsTask, extract_answer
from .trainer import PolicyTrainer
from .types import Episode
from .weight_sync import ParamArena, build_bare_model, full_tensor, sync_local


class Provisioner:
    """Hands out disjoint rank ranges of the job to roles (trainer first, then generator replicas)."""

    def __init__(self, total_gpus: int = 8):
        self.total_gpus, self.next_gpu = total_gpus, 0

    @property
    def available(self) -> int:
        return self.total_gpus - self.next_gpu

    def allocate(self, num_gpus: int) -> list[int]:
        if num_gpus > self.available:
            raise RuntimeError(f"Requested {num_gpus} GPUs but only {self.available} available "
                               f"(total={self.total_gpus}, allocated={self.next_gpu})")
        ids = list(range(self.next_gpu, self.next_gpu + num_gpus))
        self.next_gpu += num_gpus
        return ids


def _log_samples(episodes: list[Episode]) -> None:
    seen: set[str] = set()
    for ep in episodes:
        if ep.group_id in seen:
            continue
        seen.add(ep.group_id)
        got = extract_answer(ep.text)
        ok = got == int(ep.expected_answer) if ep.expected_answer else None
        logger.info(f"  [{'+' if ok else '-'}] expected={ep.expected_answer} extracted={got} reward={ep.reward:+.1f}")
        logger.info(f"       A: {ep.text[:300].replace(chr(10), ' ').strip()}")


class RLTrainer(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        model_spec: ModelSpec | None = None
        hf_assets_path: str = "./tests/assets/tokenizer"
        num_steps: int = 10
        dump_folder: str = "outputs/rl"
        batch_invariant_mode: bool = True
        num_episodes_per_step: int = 5
        log_samples: bool = False
        trainer: PolicyTrainer.Config = field(default_factory=PolicyTrainer.Config)
        generator: Generator.Config = field(default_factory=Generator.Config)
        async_mode: bool = False
        peer_weight_sync: bool = True
        """Disaggregated GPU runs: move weights with the NVLink peer-memory kernel when possible (else one arena broadcast)."""
        eval_samples: int = 20

    def __init__(self, config: Config):
        self.config = config
        self.task = SumDigitsTask(seed=42)
        self.history: list[dict] = []

    @staticmethod
    def _compute_world_size(p) -> int:
        return (p.data_parallel_replicate_degree * max(p.data_parallel_shard_degree, 1) * p.tensor_parallel_degree
                * p.pipeline_parallel_degree * p.context_parallel_degree)

    # ---- setup ------------------------------------------------------------------------------------------------
    def setup(self, device=None, tokenizer=None):
        from torchtitan_b200.components.tokenizer import HuggingFaceTokenizer

        c = self.config
        self.tokenizer = tokenizer or HuggingFaceTokenizer(tokenizer_path=c.hf_assets_path)
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.trainer_world = self._compute_world_size(c.trainer.parallelism)
        self.colocated = world == self.trainer_world
        self.system_prompt = self.task.get_system_prompt()
        self.trainer = self.generator = self.arena = None
        self.trainer_group = self.all_group = None
        if self.colocated:
            self.is_trainer = self.is_generator = True
            self.gen_ranks = [0]
        else:
            prov = Provisioner(world)
            train_ranks = prov.allocate(self.trainer_world)
            self.gen_ranks = prov.allocate(prov.available)
            self.is_trainer, self.is_generator = rank in train_ranks, rank in self.gen_ranks
            self.trainer_group = dist.new_group(train_ranks)
            self.sync_group = dist.new_group([train_ranks[0]] + self.gen_ranks)
        logger.info(f"{len(self.gen_ranks)} generator GPUs + {self.trainer_world} trainer GPUs"
                    f"{' (colocated)' if self.colocated else ''}")
        if not self.colocated and not self.is_trainer:
            # take part in the creation of the trainer's process groups (a collective of the whole job)
            PolicyTrainer.make_parallel_dims(c.trainer, self.trainer_world, train_ranks).build_mesh()
        if self.is_trainer:
            self.trainer = PolicyTrainer(c.trainer, model_spec=c.model_spec, batch_invariant_mode=c.batch_invariant_mode,
                                         hf_assets_path=c.hf_assets_path, device=device, group=self.trainer_group,
                                         ranks=None if self.colocated else train_ranks)
        self.peer_sync = None
        if not self.colocated and c.peer_weight_sync and torch.cuda.is_available() and c.generator.model_dtype == "bfloat16":
            self.peer_sync = self._maybe_peer_sync(train_ranks, device)
        if self.is_generator:
            self.generator = Generator(c.generator, model_spec=c.model_spec, model_path=c.hf_assets_path,
                                       batch_invariant_mode=c.batch_invariant_mode, tokenizer=self.tokenizer, device=device)
            self.arena = ParamArena(self.generator.model, alloc=self.peer_sync.alloc if self.peer_sync else None)
            self.generator.arena = self.arena
        elif rank == 0 and self.peer_sync is None:
            # the first trainer rank stages the generator-layout arena that is broadcast to the replicas
            self.arena = ParamArena(build_bare_model(c.model_spec, c.generator.model_dtype, device), double_buffer=False)
        if self.peer_sync is not None and self.is_trainer:
            self.peer_sync.build_plan(self.trainer.model, self._arena_offsets)
        self.grader = Grader(self.task.reward_function)
        self._sync_weights(0)

    def _maybe_peer_sync(self, train_ranks, device):
        """One symmetric heap over all ranks of the job when every GPU can map every other one; else None (broadcast path)."""
        from torchtitan_b200.ops import native

        from torchtitan_b200.parallel.nvlink_comm import peer_memory_group_ok

        from .weight_sync import NvlinkWeightSync, arena_layout

        # FSDP (or single-rank) trainers only: tensor-parallel shards are not dim-0 slices of the full parameter
        p = self.config.trainer.parallelism
        ok = (native.available() and native.has("tt_push_cast") and p.tensor_parallel_degree == 1
              and p.pipeline_parallel_degree == 1)
        if not peer_memory_group_ok(dist.group.WORLD, extra_ok=ok):
            return None
        with torch.device("meta"):
            meta = self.config.model_spec.model.build()
        if getattr(meta, "enable_weight_tying", False):
            meta.tok_embeddings.weight = meta.output.weight
        self._arena_offsets, numel = arena_layout(meta)
        return NvlinkWeightSync(dist.group.WORLD, train_ranks, self.gen_ranks, numel, device or f"cuda:{torch.cuda.current_device()}")

    def _sync_weights(self, version: int) -> None:
        """Trainer -> generator weights. Returns the time spent (seconds, host clock around a device sync)."""
        t0 = time.perf_counter()
        if self.colocated:
            sync_local(self.trainer.model, self.arena)
        elif self.peer_sync is not None:
            if self.is_trainer:
                self.peer_sync.push()
            else:
                self.peer_sync.wait_and_flip(self.arena)
        else:
            rank = dist.get_rank()
            if self.trainer is not None:
                # every trainer rank takes part in un-sharding (collectives inside the trainer group); rank 0 keeps the result
                dst = self.arena.staging() if rank == 0 else None
                with torch.no_grad():
                    for name, p in self.trainer.model.named_parameters():
                        t = full_tensor(p)
                        if dst is not None and name in dst:
                            dst[name].copy_(t)
            if self.arena is not None:
                dist.broadcast(self.arena.halves[self.arena.inactive], src=0, group=self.sync_group)
                self.arena.flip()
        if self.generator is not None:
            self.generator.update(version)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.last_sync_s = time.perf_counter() - t0

    # ---- rollouts across generator replicas -------------------------------------------------------------------
    def _generate_local(self, prompts: list, answers: list[str] | None = None) -> list[Episode]:
        """This rank's share of a rollout (empty on pure trainer ranks). ``prompts`` are texts or token-id lists."""
        if self.generator is None or not self.is_generator:
            return []
        by_ids = bool(prompts) and not isinstance(prompts[0], str)
        gen = self.generator.generate_from_ids if by_ids else self.generator.generate
        if self.colocated:
            return gen(prompts, answers)
        k = self.gen_ranks.index(dist.get_rank())
        idx = list(range(k, len(prompts), len(self.gen_ranks)))
        eps = gen([prompts[i] for i in idx], [answers[i] for i in idx] if answers else None)
        for e in eps:   # make group ids unique across replicas
            e.group_id = f"g{k}-{e.group_id}"
        return eps

    def _gather_episodes(self, mine: list[Episode]) -> list[Episode]:
        if self.colocated:
            return mine
        gathered: list = [None] * dist.get_world_size()
        dist.all_gather_object(gathered, mine)
        return [e for part in gathered for e in (part or [])]

    def _rollout(self, prompts: list, answers: list[str] | None = None) -> list[Episode]:
        return self._gather_episodes(self._generate_local(prompts, answers))

    def _questions(self, task: SumDigitsTask, n: int):
        prompts, answers = [], []
        for _ in range(n):
            q, a = task.create_question()
            prompts.append(self.system_prompt + "\n\n" + q)
            answers.append(a)
        return prompts, answers

    def evaluate(self, num_samples: int | None = None) -> dict:
        n = num_samples or self.config.eval_samples
        prompts, answers = self._questions(SumDigitsTask(seed=99), n)
        episodes = self._rollout(prompts, answers)
        per = self.config.generator.num_samples_per_prompt
        firsts = episodes[::per][:n] if self.colocated else list({e.group_id: e for e in reversed(episodes)}.values())[:n]
        correct = sum(int(extract_answer(e.text) == int(e.expected_answer)) for e in firsts if e.expected_answer)
        fmt = sum(int(bool(re.search(r"\[ANSWER\]", e.text))) for e in firsts)
        res = {"accuracy": correct / n, "correct": correct, "total": n, "format_rate": fmt / n, "format_ok": fmt}
        logger.info(f"Eval: Accuracy={res['accuracy']:.0%} ({correct}/{n}) Format={res['format_rate']:.0%} ({fmt}/{n})")
        return res

    # ---- the loop -------------------------------------------------------------------------------------------------
    def train(self) -> list[dict]:
        c = self.config
        logger.info("Evaluating pre-training baseline...")
        pre = self.evaluate()
        logger.info(f"Starting RL training for {c.num_steps} steps")
        # async mode = one step off-policy: while the trainer ranks work on batch k, the generator ranks already produce
        # batch k + 1 with the weights of step k - 1; the blocking exchange of episodes comes after both.
        episodes = self._rollout(*self._questions(self.task, c.num_episodes_per_step)) if c.async_mode else None
        for step in range(c.num_steps):
            t0 = time.perf_counter()
            nxt_local = None
            if not c.async_mode:
                episodes = self._rollout(*self._questions(self.task, c.num_episodes_per_step))
            elif step + 1 < c.num_steps:
                nxt_local = self._generate_local(*self._questions(self.task, c.num_episodes_per_step))
            episodes = group_mean_advantages(self.grader.score(episodes))
            if c.log_samples:
                _log_samples(episodes)
            metrics = self.trainer.step(episodes) if self.trainer is not None else None
            cur = episodes
            if nxt_local is not None:
                episodes = self._gather_episodes(nxt_local)
            if not self.colocated:
                box = [metrics]
                dist.broadcast_object_list(box, src=0)
                metrics = box[0]
            self._sync_weights(metrics["policy_version"])
            dt = time.perf_counter() - t0
            lens = [len(e.token_ids) for e in cur]
            n_ok = sum(1 for e in cur if e.reward > 0)
            metrics.update(step=step, time_s=dt, weight_sync_s=getattr(self, "last_sync_s", 0.0), avg_tokens=sum(lens) / max(1, len(lens)), correct=n_ok, total=len(cur),
                           gen_tokens_per_s=sum(lens) / dt)
            self.history.append(metrics)
            logger.info(
                f"Step {step:2d} | Loss: {metrics['loss']:+.4f} | Reward: {metrics['reward_mean']:+.3f} | "
                f"Correct: {n_ok:>2}/{len(cur)} | Avg tokens: {metrics['avg_tokens']:>3.0f} | "
                f"Logprob diff: mean={metrics['logprob_diff_mean']:.4e}, max={metrics['logprob_diff_max']:.4e} | Time: {dt:.1f}s"
            )
            if not torch.isfinite(torch.tensor(metrics["loss"])):
                logger.info("ERROR: Loss is NaN/Inf! Training diverged.")
                break
        logger.info("RL Training complete")
        post = self.evaluate()
        logger.info(f"Pre-training:  Accuracy={pre['accuracy']:.0%} Format={pre['format_rate']:.0%}")
        logger.info(f"Post-training: Accuracy={post['accuracy']:.0%} Format={post['format_rate']:.0%}")
        return self.history


def main() -> None:
    import os

    from torchtitan_b200.config.manager import ConfigManager

    init_logger()
    config = ConfigManager().parse_args()
    if "RANK" in os.environ and not dist.is_initialized():
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
    rl = RLTrainer(config)
    rl.setup()
    rl.train()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
