"""Pipeline parallel: stage layout, schedule validity (no deadlock, every action once) and
numerical equality with the single-process model on 2 CPU ranks."""

import dataclasses

import pytest
import torch

from dist_utils import run_ranks
from torchtitan_b200.parallel.pp import (
    Action, build_actions, estimate_makespan, fuse_split_backward, generate_llm_fqn_per_model_part, load_csv_actions,
    stage_indices_for_rank, validate_actions,
)


def test_fqn_layout_balanced():
    parts = generate_llm_fqn_per_model_part(4, 6, 1, 1)
    assert parts[0][0] == "tok_embeddings" and parts[-1][-2:] == ["norm", "output"]
    layers = [f for p in parts for f in p if f.startswith("layers.")]
    assert layers == [f"layers.{i}" for i in range(6)]
    assert generate_llm_fqn_per_model_part(1, 2)[0] == ["tok_embeddings", "layers.0", "layers.1", "norm", "output"]
    with pytest.raises(ValueError):
        generate_llm_fqn_per_model_part(20, 2)


@pytest.mark.parametrize("schedule,pp,spr,style", [
    ("GPipe", 4, 1, "loop"), ("1F1B", 4, 1, "loop"), ("1F1B", 2, 1, "loop"), ("Interleaved1F1B", 2, 2, "loop"),
    ("Interleaved1F1B", 4, 2, "loop"), ("LoopedBFS", 2, 3, "loop"), ("ZBVZeroBubble", 2, 2, "v"), ("DualPipeV", 4, 2, "v"),
])
@pytest.mark.parametrize("n_mb", [4, 8, 5])
def test_schedules_are_complete_and_deadlock_free(schedule, pp, spr, style, n_mb):
    num_stages = pp * spr
    ranks = build_actions(schedule, pp, num_stages, n_mb, style)
    validate_actions(ranks, pp, num_stages, n_mb, style)
    for r, acts in enumerate(ranks):
        stages = stage_indices_for_rank(r, pp, num_stages, style)
        assert sorted((a.stage, a.kind, a.mb) for a in acts) == sorted(
            (s, k, m) for s in stages for k in "FB" for m in range(n_mb))


@pytest.mark.parametrize("schedule,pp,spr,style", [
    ("InterleavedZeroBubble", 4, 2, "loop"), ("InterleavedZeroBubble", 2, 3, "loop"), ("ZBVZeroBubble", 2, 2, "v"),
    ("ZBVZeroBubble", 4, 2, "v"), ("DualPipeV", 8, 2, "v"),
])
@pytest.mark.parametrize("n_mb", [4, 8, 5, 16])
def test_zero_bubble_schedules_split_the_backward(schedule, pp, spr, style, n_mb):
    num_stages = pp * spr
    split = build_actions(schedule, pp, num_stages, n_mb, style, split=True)
    validate_actions(split, pp, num_stages, n_mb, style)
    for r, acts in enumerate(split):
        stages = stage_indices_for_rank(r, pp, num_stages, style)
        assert sorted((a.stage, a.kind, a.mb) for a in acts) == sorted(
            (s, k, m) for s in stages for k in "FIW" for m in range(n_mb))
        where = {(a.stage, a.kind, a.mb): i for i, a in enumerate(acts)}
        assert all(where[(s, "W", m)] > where[(s, "I", m)] for s in stages for m in range(n_mb))
    # the weight-gradient halves are really moved: on some rank one runs after a later micro-batch's input gradient
    assert any(a.kind == "W" and any(b.kind == "I" and (b.stage, b.mb) != (a.stage, a.mb) for b in acts[i - 1:i])
               for acts in split for i, a in enumerate(acts) if i)
    whole = build_actions(schedule, pp, num_stages, n_mb, style)
    validate_actions(whole, pp, num_stages, n_mb, style)
    assert estimate_makespan(split, num_stages)[0] <= estimate_makespan(whole, num_stages)[0]
    if n_mb >= 2 * pp:                                   # the idle share of a step, forward 1 / backward 2 units
        assert estimate_makespan(split, num_stages)[1] < 0.15
    fused = fuse_split_backward(split)
    validate_actions(fused, pp, num_stages, n_mb, style)
    assert all(a.kind in "FB" for acts in fused for a in acts)


def test_schedule_checks_reject_a_weight_step_before_its_input_step(tmp_path):
    path = tmp_path / "sched.csv"
    path.write_text("0F0,0F1,0I0,0W0,0I1,0W1\n1F0,1I0,1F1,1I1,1W0,1W1\n")
    ranks = load_csv_actions(str(path))
    assert ranks[1][-1] == Action(1, "W", 1) and ranks[0][2].kind == "I"
    validate_actions(ranks, 2, 2, 2, "loop")
    bad = [ranks[0], [Action(1, "F", 0), Action(1, "W", 0), Action(1, "I", 0), Action(1, "F", 1), Action(1, "I", 1), Action(1, "W", 1)]]
    with pytest.raises(RuntimeError, match="comes before"):
        validate_actions(bad, 2, 2, 2, "loop")
    with pytest.raises(RuntimeError, match="without a weight-gradient step"):
        validate_actions([ranks[0], ranks[1][:-1]], 2, 2, 2, "loop")


def _worker(rank, world, schedule, overlap=False):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.config import ActivationCheckpointConfig, CompileConfig, ParallelismConfig, TrainingConfig
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.models.llama3.parallelize import parallelize_llama
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.pp import pipeline_llm
    from torchtitan_b200.protocols.model_converter import ModelConvertersContainer

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=1, pp=world, ep=1, etp=1, world_size=world)
    cfg = dataclasses.replace(llama3_configs["debugmodel_gqa"], n_layers=4)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=32)
    torch.manual_seed(3)
    ref = cfg.build()
    ref.init_weights()
    B = 4
    x = torch.randint(0, cfg.vocab_size, (B, 33))
    inp, lab = x[:, :-1], x[:, 1:]
    training = TrainingConfig(local_batch_size=B, seq_len=32)
    par = ParallelismConfig(pipeline_parallel_degree=world, pipeline_parallel_schedule=schedule, pipeline_parallel_microbatch_size=1)
    sched, parts, first, last = pipeline_llm(
        ref, parallel_dims=pd, training=training, model_converters=ModelConvertersContainer.Config(), parallelism=par,
        compile_config=CompileConfig(), ac_config=ActivationCheckpointConfig(mode="none"), dump_folder="/tmp",
        device=torch.device("cpu"), model_config=cfg, parallelize_fn=parallelize_llama, loss_fn=cross_entropy_loss,
    )
    if overlap:
        # whole backward steps, neighbours of different micro-batches merged into slots that run both halves on two threads
        sched.all_actions = build_actions(schedule, world, 2 * world, B, "v", split=False, overlap=True)
        validate_actions(sched.all_actions, world, 2 * world, B, "v")
        from torchtitan_b200.ops.wgrad_store import WeightGradStore

        WeightGradStore.enabled = False
    losses = [] if last else None
    scale = torch.tensor(1.0 / lab.numel())
    if first:
        sched.step(inp, target=lab if last else None, losses=losses, loss_scale=scale)
    else:
        sched.step(target=lab if last else None, losses=losses, loss_scale=scale)
    ref_loss = cross_entropy_loss(ref(inp), lab) / lab.numel()
    ref_loss.backward()
    out = {"ref": ref_loss.item(), "loss": float(torch.stack(losses).sum()) if last else None, "grad_err": 0.0}
    ref_grads = dict(ref.named_parameters())
    for part in parts:
        for name, p in part.named_parameters():
            out["grad_err"] = max(out["grad_err"], (p.grad - ref_grads[name].grad).abs().max().item())
    # forward-only evaluation through the same stages
    ev = [] if last else None
    if first:
        sched.eval(inp, target=lab if last else None, losses=ev)
    else:
        sched.eval(target=lab if last else None, losses=ev)
    out["eval"] = float(torch.stack(ev).sum()) / lab.numel() if last else None
    out["kinds"] = "".join(sorted({a.kind for a in sched.all_actions[rank]}))
    return out


@pytest.mark.parametrize("schedule", ["1F1B", "Interleaved1F1B", "InterleavedZeroBubble", "ZBVZeroBubble", "DualPipeV"])
def test_pp2_matches_single_process(tmp_path, schedule):
    res = run_ranks(_worker, 2, schedule, tmp_path=tmp_path)
    # pipeline-only stages own their gradients, so the zero-bubble schedules run with separate I / W steps
    assert all(o["kinds"] == ("FIW" if "Zero" in schedule or schedule == "DualPipeV" else "BF") for o in res), res
    got = [o for o in res if o["loss"] is not None]
    assert got, res
    for o in got:
        assert abs(o["loss"] - o["ref"]) < 1e-5, o
        assert abs(o["eval"] - o["ref"]) < 1e-5, o
    assert max(o["grad_err"] for o in res) < 1e-5, res


def test_overlapped_forward_backward_slots_match_single_process(tmp_path):
    """DualPipeV slots that run a forward and a backward of different micro-batches on two threads: same loss and
    gradients as the single-process model."""
    res = run_ranks(_worker, 2, "DualPipeV", True, tmp_path=tmp_path)
    assert any("O" in o["kinds"] for o in res), res
    got = [o for o in res if o["loss"] is not None]
    for o in got:
        assert abs(o["loss"] - o["ref"]) < 1e-5, o
    assert max(o["grad_err"] for o in res) < 1e-5, res


def test_overlap_baton_alternates_at_yield_points():
    from torchtitan_b200.parallel.overlap import active, run_overlapped, yield_point

    log = []

    def piece(name, n):
        def run():
            assert active()
            for i in range(n):
                log.append(f"{name}{i}")
                yield_point()
            return name
        return run

    assert run_overlapped(piece("a", 3), piece("b", 5)) == ("a", "b")
    assert log == ["a0", "b0", "a1", "b1", "a2", "b2", "b3", "b4"] and not active()
    with pytest.raises(ZeroDivisionError):
        run_overlapped(lambda: 1 / 0, piece("c", 2))


def test_overlapped_slot_syntax_and_checks(tmp_path):
    path = tmp_path / "s.csv"
    path.write_text("0F0,0F1,0B0,0B1\n1F0,1F1+1B0,1B1\n")
    ranks = load_csv_actions(str(path))
    assert ranks[1][1] == Action(1, "O", 1, ("B", 1, 0)) and [p.kind for p in ranks[1][1].parts()] == ["F", "B"]
    validate_actions(ranks, 2, 2, 2, "loop")
    # both halves wait for their inputs before either sends: pairing 0F1 with 0B0 would wait for a gradient that needs 0F1... of
    # the same rank's later work only if the micro-batches were equal; an equal pair is rejected as a deadlock
    bad = [[Action(0, "F", 0), Action(0, "O", 1, ("B", 0, 1))], [Action(1, "F", 0), Action(1, "B", 0), Action(1, "F", 1), Action(1, "B", 1)]]
    with pytest.raises(RuntimeError):
        validate_actions(bad, 2, 2, 2, "loop")


def test_keyword_arguments_are_cut_per_micro_batch():
    """Mask records travel to every stage as keyword arguments; each micro-batch must see its own rows."""
    from torchtitan_b200.models.common.attention import AttentionMasks
    from torchtitan_b200.parallel.pp import _batch_size_hint, _micro_batch_of

    doc = torch.arange(4 * 6).view(4, 6)
    masks = AttentionMasks(doc_ids=doc, cu_seqlens=torch.tensor([0, 24]), max_seqlen=24, window=3)
    kw = {"attention_masks": {"rope": masks, "nope": AttentionMasks()}, "positions": torch.arange(6).view(1, 6), "flag": True}
    assert _batch_size_hint(kw) == 4
    got = [{k: _micro_batch_of(v, 2, m, 4) for k, v in kw.items()} for m in range(2)]
    assert torch.equal(got[1]["attention_masks"]["rope"].doc_ids, doc[2:]) and got[1]["attention_masks"]["rope"].window == 3
    assert got[0]["attention_masks"]["rope"].cu_seqlens is None            # packed boundaries no longer describe the rows
    assert got[0]["attention_masks"]["nope"].doc_ids is None
    assert got[0]["positions"].shape == (1, 6) and got[0]["flag"] is True
    assert _micro_batch_of(masks, 1, 0, 4) is masks


def _fsdp_worker(rank, world, schedule, ac_mode):
    """pp 2 x dp_shard 2: every pipeline stage is wrapped in FSDP units, the backward steps are split, and the units'
    gradient reductions run at the end of the weight-gradient steps."""
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.config import ActivationCheckpointConfig, CompileConfig, ParallelismConfig, TrainingConfig
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.models.llama3.parallelize import parallelize_llama
    from torchtitan_b200.parallel import ParallelDims, fsdp
    from torchtitan_b200.parallel.pp import pipeline_llm
    from torchtitan_b200.protocols.model_converter import ModelConvertersContainer

    pd = ParallelDims(dp_replicate=1, dp_shard=2, cp=1, tp=1, pp=2, ep=1, etp=1, world_size=world)
    dp_rank = pd.coordinate("fsdp", rank)
    cfg = dataclasses.replace(llama3_configs["debugmodel_gqa"], n_layers=4)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=32)
    torch.manual_seed(3)
    ref = cfg.build()
    ref.init_weights()
    full_state = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    B = 4
    x_all = torch.randint(0, cfg.vocab_size, (2 * B, 33), generator=torch.Generator().manual_seed(9))
    x = x_all[dp_rank * B:(dp_rank + 1) * B]                    # the two data-parallel ranks see different rows
    inp, lab = x[:, :-1], x[:, 1:]
    training = TrainingConfig(local_batch_size=B, seq_len=32, mixed_precision_param="float32", mixed_precision_reduce="float32")
    par = ParallelismConfig(pipeline_parallel_degree=2, data_parallel_shard_degree=2, pipeline_parallel_schedule=schedule,
                            pipeline_parallel_microbatch_size=1)
    model = cfg.build()
    model.init_weights()                                         # also builds the rotary table, which is not part of the state
    model.load_state_dict(full_state)
    sched, parts, first, last = pipeline_llm(
        model, parallel_dims=pd, training=training, model_converters=ModelConvertersContainer.Config(), parallelism=par,
        compile_config=CompileConfig(), ac_config=ActivationCheckpointConfig(mode=ac_mode), dump_folder="/tmp",
        device=torch.device("cpu"), model_config=cfg, parallelize_fn=parallelize_llama, loss_fn=cross_entropy_loss,
    )
    for part in parts:
        assert fsdp.fsdp_units(part)
        fsdp.materialize(part)
    losses = [] if last else None
    scale = torch.tensor(1.0 / (2 * lab.numel()))                # per global token: the units sum over data-parallel ranks
    for _ in range(2):                                           # a second step accumulates onto the first one's gradients
        if first:
            sched.step(inp, target=lab if last else None, losses=losses, loss_scale=scale)
        else:
            sched.step(target=lab if last else None, losses=losses, loss_scale=scale)
    inp_all, lab_all = x_all[:, :-1], x_all[:, 1:]
    ref_loss = cross_entropy_loss(ref(inp_all), lab_all) / lab_all.numel()
    (2 * ref_loss).backward()                                    # two identical steps, gradients add up
    ref_grads = dict(ref.named_parameters())
    err = 0.0
    for part in parts:
        for name, p in part.named_parameters():
            g = p.grad.full_tensor() if hasattr(p.grad, "full_tensor") else p.grad
            err = max(err, (g - ref_grads[name].grad).abs().max().item())
    return {"grad_err": err, "kinds": "".join(sorted({a.kind for a in sched.all_actions[pd.coordinate("pp", rank)]})),
            "loss": float(torch.stack(losses).sum()) if last else None}


@pytest.mark.parametrize("schedule,ac_mode", [("ZBVZeroBubble", "none"), ("InterleavedZeroBubble", "full"), ("DualPipeV", "selective")])
def test_split_backward_under_fsdp_matches_single_process(tmp_path, schedule, ac_mode):
    res = run_ranks(_fsdp_worker, 4, schedule, ac_mode, tmp_path=tmp_path)
    assert all("I" in o["kinds"] and "W" in o["kinds"] and "B" not in o["kinds"] for o in res), res
    assert max(o["grad_err"] for o in res) < 1e-5, res
    assert any(o["loss"] is not None for o in res)
