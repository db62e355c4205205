"""GRPO step-time benchmark on one node.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m torchtitan_b200.experiments.rl.bench_grpo --trainer-gpus 4 --steps 3 --warmup 1

Workload (synthetic, random-init weights): a Qwen3-1.7B-shaped policy (dim 2048, 28 layers, 16 Q / 8 KV heads,
head_dim 128, FFN 6144, vocab 151936, tied embeddings) in bf16; per step ``--prompts`` prompts of random token ids in
[1000, 150000) with lengths uniform in [128, 512] (seed 0), ``--samples`` samples each at temperature 1.0, up to
``--max-new`` new tokens through the paged-KV engine; reward = fraction of generated ids divisible by 7, plus 1.0 when
the completion has at most 512 tokens; group-normalised advantages; token-level PPO clip 0.2 without a KL term; full
bf16 weight sync trainer -> generators after every optimizer step; one-step-off-policy asynchronous rollouts.
The first ``--trainer-gpus`` ranks train with FSDP, the remaining ranks are generator replicas. Rank 0 prints one JSON
line: seconds per GRPO step (wall clock between device synchronisations, maximum over ranks), generated tokens per
second, and weight-sync milliseconds. With one rank the roles are colocated.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import time

import torch
import torch.distributed as dist


def _reward(ep) -> float:
    ids = ep.token_ids
    frac = sum(1 for t in ids if t % 7 == 0) / max(1, len(ids))
    return frac + (1.0 if len(ids) <= 512 else 0.0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--trainer-gpus", type=int, default=0, help="0 = half of the ranks (all of them when colocated)")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--prompts", type=int, default=64)
    ap.add_argument("--samples", type=int, default=8)
    ap.add_argument("--max-new", type=int, default=1024)
    ap.add_argument("--flavor", default="1.7B")
    ap.add_argument("--sync", default="peer", choices=["peer", "broadcast"])
    ap.add_argument("--no-cudagraph", action="store_true")
    a = ap.parse_args()

    from torchtitan_b200.experiments.rl.config_registry import rl_grpo_qwen3_debug
    from torchtitan_b200.experiments.rl.grader import group_mean_advantages
    from torchtitan_b200.experiments.rl.simple_grpo_sum_digits import RLTrainer
    from torchtitan_b200.models.qwen3 import model_registry
    from torchtitan_b200.tools.logging import init_logger

    init_logger()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ntrain = a.trainer_gpus or max(1, world // 2)
    cfg = rl_grpo_qwen3_debug()
    cfg.model_spec = model_registry(a.flavor)
    cfg.trainer.parallelism.data_parallel_shard_degree = ntrain if world > 1 else 1
    cfg.trainer.objective, cfg.trainer.kl_coef = "dapo", 0.0
    cfg.trainer.clip_low = cfg.trainer.clip_high = 0.2
    cfg.trainer.optimizer.lr = 1e-6
    cfg.generator.num_samples_per_prompt = a.samples
    cfg.generator.sampling.temperature, cfg.generator.sampling.top_p, cfg.generator.sampling.max_tokens = 1.0, 1.0, a.max_new
    cfg.generator.compile.cudagraph_mode = "none" if a.no_cudagraph else "piecewise"
    if a.no_cudagraph:
        cfg.generator.compile.backend = "none"
    cfg.generator.seed = 1234 + rank
    # KV cache sized for the benchmark instead of "all free memory": sequences of this replica x longest possible length
    n_gen = 1 if world == 1 else world - ntrain
    seqs = -(-a.prompts // n_gen) * a.samples
    cfg.generator.max_kv_blocks = int(seqs * (512 + a.max_new + 32) / cfg.generator.kv_block_size * 1.1) + 64
    cfg.peer_weight_sync = a.sync == "peer"
    cfg.async_mode = True

    class _Tok:   # token ids in, token ids out: the benchmark never touches text
        eos_id = None

        def decode(self, ids):
            return ""

    rl = RLTrainer(cfg)
    rl.setup(tokenizer=_Tok())
    rng = random.Random(0)

    def make_prompts():
        return [[rng.randrange(1000, 150000) for _ in range(rng.randint(128, 512))] for _ in range(a.prompts)]

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    times, syncs, gen_tokens = [], [], []
    episodes = rl._rollout(make_prompts())
    total_steps = a.warmup + a.steps
    for step in range(total_steps):
        sync()
        t0 = time.perf_counter()
        # generator ranks start batch k + 1 (weights of step k - 1) while trainer ranks run step k
        nxt_local = rl._generate_local(make_prompts()) if step + 1 < total_steps else None
        for e in episodes:
            e.reward = _reward(e)
        group_mean_advantages(episodes, normalize_std=True)
        metrics = rl.trainer.step(episodes) if rl.trainer is not None else None
        cur = episodes
        if nxt_local is not None:
            episodes = rl._gather_episodes(nxt_local)
        if not rl.colocated:
            box = [metrics]
            dist.broadcast_object_list(box, src=0)
            metrics = box[0]
        rl._sync_weights(metrics["policy_version"])
        sync()
        dt = time.perf_counter() - t0
        if step >= a.warmup:
            times.append(dt)
            syncs.append(rl.last_sync_s)
            gen_tokens.append(sum(len(e.token_ids) for e in cur))
    t = torch.tensor([sum(times) / len(times), max(syncs)], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        from torchtitan_b200.ops import native

        print(json.dumps({
            "metric": "grpo_step_seconds", "value": t[0].item(), "unit": "s/step", "higher_is_better": False, "n_gpus": world,
            "trainer_gpus": ntrain if world > 1 else 1, "generator_gpus": world - ntrain if world > 1 else 1,
            "weight_sync_ms": t[1].item() * 1e3, "weight_sync_path": ("peer-memory kernel" if rl.peer_sync is not None else
                                                                      ("local cast/copy" if rl.colocated else "arena broadcast")),
            "generated_tokens_per_step": sum(gen_tokens) / len(gen_tokens),
            "generated_tokens_per_s": sum(gen_tokens) / sum(times), "steps": a.steps, "warmup": a.warmup,
            "config": {"model": f"Qwen3-{a.flavor} shape, random init, bf16", "prompts": a.prompts, "samples": a.samples,
                       "max_new_tokens": a.max_new, "objective": "token-level PPO clip 0.2, no KL, group-normalised advantages",
                       "async": "one step off-policy", "data": "synthetic token ids (seed 0)"},
            "loss": metrics["loss"], "kernel_errors": native.kernel_errors(),
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
