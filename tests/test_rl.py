"""RL experiment on CPU: task/grader, sampler and paged attention definitions, engine-vs-trainer
log-probability agreement, one colocated GRPO run."""

import dataclasses
import os

import pytest
import torch


def test_sum_digits_task_and_rewards():
    from torchtitan_b200.experiments.rl.sum_digits import SumDigitsTask, extract_answer

    t = SumDigitsTask(seed=1)
    q, a = t.create_question()
    nums = [int(x) for x in q[q.index("[") + 1 : q.index("]")].split(",")]
    assert int(a) == sum(int(d) for n in nums for d in str(n))
    assert SumDigitsTask(seed=1).create_question() == (q, a)
    assert extract_answer("so 3 + 4 = 7\n[ANSWER] 7") == 7
    assert extract_answer("The answer is 12.") == 12
    assert extract_answer("i think 5 then 9") == 9 and extract_answer("none") is None
    r = t.reward_function(["[ANSWER] 7", "x [ANSWER] 7 trailing", "[ANSWER] 8"], "7")
    assert r.tolist() == pytest.approx([1.2, 1.0, -1.0])


def test_group_mean_advantages():
    from torchtitan_b200.experiments.rl.grader import group_mean_advantages
    from torchtitan_b200.experiments.rl.types import Episode

    eps = [Episode(0, [1], "", [2], [0.0], reward=r, group_id=g) for r, g in ((1, "a"), (-1, "a"), (1, "b"), (1, "b"))]
    group_mean_advantages(eps)
    assert [e.advantage for e in eps] == [1.0, -1.0, 0.0, 0.0]


def test_sampler_definition():
    from torchtitan_b200.ops.serving import sample_top_p

    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).repeat(3, 1)
    tok, lp = sample_top_p(logits, 0.0, 1.0, torch.zeros(3))
    assert tok.tolist() == [0, 0, 0] and torch.allclose(lp, torch.log_softmax(logits, -1)[:, 0])
    # top_p small enough keeps only the best token whatever the draw
    tok, _ = sample_top_p(logits, 1.0, 0.5, torch.tensor([0.0, 0.5, 0.999]))
    assert tok.tolist() == [0, 0, 0]
    # top_p = 1: plain multinomial, the draw walks the CDF in index order
    p = torch.softmax(logits[0], -1)
    tok, lp = sample_top_p(logits, 1.0, 1.0, torch.tensor([0.0, float(p[0]) + 1e-3, 0.9999]))
    assert tok.tolist() == [0, 1, 3]
    rev = logits.flip(-1)
    tok, _ = sample_top_p(rev, 1.0, 1.0, torch.tensor([0.0, float(p[3]) + 1e-3, 0.9999]))
    assert tok.tolist() == [0, 1, 3]
    assert torch.allclose(lp, torch.log_softmax(logits, -1)[0, tok])


def test_paged_decode_definition_matches_dense():
    from torchtitan_b200.ops import reference
    from torchtitan_b200.ops.serving import kv_cache_write, paged_attention_decode

    torch.manual_seed(0)
    B, H, Hkv, D, bs = 3, 4, 2, 16, 4
    lens = [5, 9, 12]
    kc, vc = torch.zeros(16, bs, Hkv, D), torch.zeros(16, bs, Hkv, D)
    tables = torch.zeros(B, 3, dtype=torch.int32)
    perm = torch.randperm(16).tolist()
    outs = []
    q = torch.randn(B, H, D)
    for b, n in enumerate(lens):
        blks = [perm.pop() for _ in range((n + bs - 1) // bs)]
        tables[b, : len(blks)] = torch.tensor(blks)
        k, v = torch.randn(n, Hkv, D), torch.randn(n, Hkv, D)
        slots = torch.tensor([blks[t // bs] * bs + t % bs for t in range(n)], dtype=torch.int32)
        kv_cache_write(kc, vc, k, v, slots)
        o = reference.attention(q[b].view(1, 1, H, D), k.unsqueeze(0), v.unsqueeze(0), causal=False, scale=D**-0.5)
        outs.append(o.view(H, D))
    got = paged_attention_decode(q, kc, vc, tables, torch.tensor(lens, dtype=torch.int32), D**-0.5)
    assert torch.allclose(got, torch.stack(outs), atol=1e-5)


def _debug_spec():
    from torchtitan_b200.models.qwen3 import model_registry

    spec = model_registry("debugmodel")
    spec.model = dataclasses.replace(spec.model, n_layers=2)
    spec.model.rope = dataclasses.replace(spec.model.rope, max_seq_len=512)
    return spec


def test_engine_logprobs_match_trainer_recompute():
    from torchtitan_b200.experiments.rl.generator import Generator, SamplingConfig
    from torchtitan_b200.experiments.rl.losses import compute_token_log_probs_packed

    torch.manual_seed(0)
    spec = _debug_spec()
    gen = Generator(Generator.Config(num_samples_per_prompt=3, seed=7, max_kv_blocks=256, kv_block_size=4,
                                     sampling=SamplingConfig(temperature=1.0, top_p=0.9, max_tokens=12)),
                    model_spec=spec, device="cpu")
    prompts = [[1, 5, 9, 12, 7], [3, 4, 100, 200, 300, 17, 21, 9, 2]]
    eps = gen.generate_from_ids(prompts, ["1", "2"])
    assert len(eps) == 6 and eps[0].group_id == eps[2].group_id != eps[3].group_id
    assert all(len(e.token_ids) == len(e.token_log_probs) <= 12 for e in eps)
    assert gen.engine.cache.alloc.available == 256           # every block returned
    lps = compute_token_log_probs_packed(gen.model, [e.prompt_token_ids for e in eps], [e.token_ids for e in eps], "cpu")
    for e, lp in zip(eps, lps):
        assert torch.allclose(torch.tensor(e.token_log_probs), lp, atol=2e-5), (e.token_log_probs, lp)
    # samples of one prompt are not all identical at temperature 1
    assert len({tuple(e.token_ids) for e in eps[:3]}) > 1


def test_param_arena_double_buffer():
    from torchtitan_b200.experiments.rl.weight_sync import ParamArena, sync_local

    spec = _debug_spec()
    a, b = spec.model.build(), spec.model.build()
    a.init_weights()
    b.init_weights()
    arena = ParamArena(b)
    before = {n: p.clone() for n, p in b.named_parameters()}
    ptr0 = b.output.weight.data_ptr()
    sync_local(a, arena)
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.equal(p, q), n
    assert b.output.weight.data_ptr() != ptr0 and arena.active == 1
    assert any(not torch.equal(before[n], p) for n, p in b.named_parameters())


def test_colocated_grpo_two_steps(tmp_path):
    from torchtitan_b200.experiments.rl.config_registry import rl_grpo_qwen3_debug
    from torchtitan_b200.experiments.rl.simple_grpo_sum_digits import RLTrainer

    cfg = rl_grpo_qwen3_debug()
    cfg.model_spec = _debug_spec()
    cfg.num_steps, cfg.num_episodes_per_step, cfg.eval_samples = 2, 2, 2
    cfg.generator.num_samples_per_prompt = 2
    cfg.generator.sampling.max_tokens = 6
    cfg.generator.max_kv_blocks = 512
    cfg.generator.seed = 0
    cfg.trainer.training.dtype = "float32"
    cfg.hf_assets_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "assets", "tokenizer")
    rl = RLTrainer(cfg)
    rl.setup(device="cpu")
    w0 = rl.generator.model.output.weight.clone()
    hist = rl.train()
    assert len(hist) == 2 and all(h["loss"] == h["loss"] for h in hist)
    assert hist[0]["logprob_diff_max"] < 1e-4        # generator and trainer agree before the first update
    assert hist[-1]["policy_version"] == 2 and rl.generator.policy_version == 2
    assert not torch.equal(w0, rl.generator.model.output.weight)   # weights reached the generator
    assert torch.equal(rl.generator.model.output.weight, rl.trainer.model.output.weight.to(w0.dtype))


def _disagg_worker(rank, world, ntrain=1, tp=1):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.experiments.rl.config_registry import rl_grpo_qwen3_debug
    from torchtitan_b200.experiments.rl.simple_grpo_sum_digits import RLTrainer

    cfg = rl_grpo_qwen3_debug()
    cfg.model_spec = _debug_spec()
    cfg.num_steps, cfg.num_episodes_per_step, cfg.eval_samples = 2, 2, 2
    cfg.generator.num_samples_per_prompt = 2
    cfg.generator.sampling.max_tokens = 5
    cfg.generator.max_kv_blocks = 512
    cfg.generator.seed = rank
    cfg.trainer.training.dtype = "float32"
    cfg.async_mode = True
    cfg.trainer.parallelism.data_parallel_shard_degree = ntrain // tp
    cfg.trainer.parallelism.tensor_parallel_degree = tp
    cfg.hf_assets_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "assets", "tokenizer")
    rl = RLTrainer(cfg)
    rl.setup(device="cpu")
    hist = rl.train()
    out = {"steps": len(hist), "version": hist[-1]["policy_version"], "is_trainer": rl.trainer is not None,
           "is_generator": rl.generator is not None, "sync_s": hist[-1]["weight_sync_s"]}
    if rl.generator is not None:
        out["gen_version"] = rl.generator.policy_version
        out["w"] = rl.generator.model.output.weight.detach().clone()
    if rl.trainer is not None:
        from torchtitan_b200.experiments.rl.weight_sync import full_tensor

        out["w"] = full_tensor(rl.trainer.model.output.weight).detach().clone()
    return out


def test_disaggregated_async_grpo_three_ranks(tmp_path):
    """1 trainer rank + 2 generator replicas over gloo: episodes are gathered, weights reach every replica."""
    from dist_utils import run_ranks

    res = run_ranks(_disagg_worker, 3, tmp_path=tmp_path)
    assert res[0]["is_trainer"] and not res[0]["is_generator"]
    assert all(r["is_generator"] and not r["is_trainer"] for r in res[1:])
    assert all(r["steps"] == 2 and r["version"] == 2 for r in res)
    for r in res[1:]:
        assert r["gen_version"] == 2 and torch.equal(r["w"], res[0]["w"])


@pytest.mark.parametrize("objective", ["grpo", "dapo"])
def test_microbatched_policy_step_equals_full_batch(objective):
    from torchtitan_b200.experiments.rl.trainer import PolicyTrainer
    from torchtitan_b200.experiments.rl.types import Episode

    def make(limit):
        torch.manual_seed(0)
        cfg = PolicyTrainer.Config(objective=objective, max_tokens_per_microbatch=limit)
        cfg.training.dtype = "float32"
        cfg.training.max_norm = 1e9
        cfg.optimizer.lr = 0.0
        return PolicyTrainer(cfg, model_spec=_debug_spec(), device="cpu")

    g = torch.Generator().manual_seed(1)
    eps = []
    for i in range(5):
        p = torch.randint(1, 2000, (int(torch.randint(4, 9, (1,), generator=g)),), generator=g).tolist()
        t = torch.randint(1, 2000, (int(torch.randint(3, 12, (1,), generator=g)),), generator=g).tolist()
        eps.append(Episode(0, p, "", t, [-7.0] * len(t), reward=float(i % 2), group_id=str(i // 2), advantage=float(i) - 2.0))
    a, b = make(10**6), make(24)
    ma, mb = a.step(eps), b.step(eps)
    assert abs(ma["loss"] - mb["loss"]) < 1e-5 and abs(ma["grad_norm"] - mb["grad_norm"]) < 1e-4 * max(1.0, ma["grad_norm"])
    for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
        if p.grad is not None:
            assert torch.allclose(p.grad, q.grad, atol=1e-6, rtol=1e-4), n


def test_disaggregated_fsdp_trainer_subgroup(tmp_path):
    """2 FSDP trainer ranks (a sub-group of the job) + 1 generator rank."""
    from dist_utils import run_ranks

    res = run_ranks(_disagg_worker, 3, 2, tmp_path=tmp_path)
    assert [r["is_trainer"] for r in res] == [True, True, False]
    assert all(r["steps"] == 2 and r["version"] == 2 for r in res)
    assert torch.equal(res[0]["w"], res[1]["w"]) and torch.equal(res[2]["w"], res[0]["w"])


def test_disaggregated_tensor_parallel_trainer(tmp_path):
    """2 tensor-parallel trainer ranks + 1 generator: the generator receives the FULL weights, reassembled from the shards
    (the layout of the reference's default RL configurations: trainer TP 2)."""
    from dist_utils import run_ranks

    res = run_ranks(_disagg_worker, 3, 2, 2, tmp_path=tmp_path)
    assert [r["is_trainer"] for r in res] == [True, True, False]
    assert all(r["steps"] == 2 and r["version"] == 2 for r in res)
    assert res[2]["w"].shape == res[0]["w"].shape and torch.equal(res[2]["w"], res[0]["w"]) and torch.equal(res[0]["w"], res[1]["w"])


def _policy_step_worker(rank, world, tp):
    import torch.distributed as dist

    if world > 1:
        dist.init_process_group("gloo")
    from torchtitan_b200.experiments.rl.trainer import PolicyTrainer
    from torchtitan_b200.experiments.rl.types import Episode
    from torchtitan_b200.experiments.rl.weight_sync import full_tensor

    torch.manual_seed(0)
    cfg = PolicyTrainer.Config(objective="grpo")
    cfg.training.dtype = "float32"
    cfg.training.max_norm = 1e9
    cfg.optimizer.lr = 1e-3
    cfg.parallelism.tensor_parallel_degree = tp
    cfg.parallelism.data_parallel_shard_degree = world // tp
    tr = PolicyTrainer(cfg, model_spec=_debug_spec(), device="cpu")
    # identical starting weights on every layout: take them from a seeded single-process model
    torch.manual_seed(11)
    src = _debug_spec().model.build()
    src.init_weights()
    from torchtitan_b200.components.checkpoint import ModelWrapper

    for model in (tr.model, tr.ref_model):
        sd = ModelWrapper(model).state_dict()
        with torch.no_grad():
            for k, v in sd.items():
                if hasattr(v, "device_mesh"):
                    from torch.distributed.tensor import distribute_tensor

                    v._local_tensor.copy_(distribute_tensor(src.state_dict()[k], v.device_mesh, v.placements)._local_tensor)
                else:
                    v.copy_(src.state_dict()[k])
        from torchtitan_b200.parallel import fsdp

        for u in fsdp.fsdp_units(model):
            u.mark_params_updated()
    g = torch.Generator().manual_seed(1)
    eps = []
    for i in range(4):
        p = torch.randint(1, 2000, (6,), generator=g).tolist()
        t = torch.randint(1, 2000, (7,), generator=g).tolist()
        eps.append(Episode(0, p, "", t, [-7.0] * len(t), reward=float(i % 2), group_id=str(i // 2), advantage=float(i) - 1.5))
    m = tr.step(eps)
    return {"loss": m["loss"], "grad_norm": m["grad_norm"], "w": full_tensor(tr.model.layers["0"].attention.wq.weight).clone()}


def test_tensor_parallel_policy_step_matches_single_process(tmp_path):
    from dist_utils import run_ranks

    one = _policy_step_worker(0, 1, 1)
    for o in run_ranks(_policy_step_worker, 2, 2, tmp_path=tmp_path):
        assert abs(o["loss"] - one["loss"]) < 1e-5, (o["loss"], one["loss"])
        assert abs(o["grad_norm"] - one["grad_norm"]) < 1e-4 * max(1.0, one["grad_norm"])
        assert torch.allclose(o["w"], one["w"], atol=1e-6)


def test_plan_microbatches_gives_every_rank_the_same_count():
    """Reference: torchtitan/experiments/rl/actors/trainer.py (micro-batching of a rank's episodes). With a sharded
    model every forward is a collective, so ranks with less to do split or repeat micro-batches."""
    from torchtitan_b200.experiments.rl.trainer import plan_microbatches

    lens = [[100, 100, 100, 100], [10, 10, 10, 10], [390]]
    plans = [plan_microbatches(lens, r, cap=200) for r in range(3)]
    assert plans[0] == ([[0, 1], [2, 3]], 2)
    assert plans[1] == ([[0, 1], [2, 3]], 2)             # one greedy group, split in two
    assert plans[2] == ([[0], [0]], 1)                   # nothing to split: a zero-weight repeat
    for r, (groups, n_real) in enumerate(plans):
        assert sorted(j for g in groups[:n_real] for j in g) == list(range(len(lens[r])))
    with pytest.raises(ValueError):
        plan_microbatches([[1], []], 1, cap=8)
