"""The sharded data-parallel runtime, activation checkpointing and the optimizer container on CPU (gloo ranks): sharded
training must reproduce single-process training (model: the reference's integration features FSDP / HSDP / DDP and
tests/unit_tests/test_activation_checkpoint.py, test_train_spec.py optimizer-container checks)."""

import copy

import pytest
import torch
import torch.nn as nn

from dist_utils import run_ranks


class _Block(nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.w1 = nn.Linear(d, h, bias=False)
        self.w2 = nn.Linear(h, d, bias=True)

    def forward(self, x):
        return x + self.w2(torch.nn.functional.silu(self.w1(self.norm(x))))


class _Net(nn.Module):
    def __init__(self, d=24, h=40, n=3, vocab=50):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)
        self.layers = nn.ModuleDict({str(i): _Block(d, h) for i in range(n)})
        self.out = nn.Linear(d, vocab, bias=False)
        self.scalar = nn.Parameter(torch.tensor(0.5))          # a 0-dim parameter rides along replicated

    def forward(self, tok):
        x = self.emb(tok)
        for b in self.layers.values():
            x = b(x)
        return self.out(x) * self.scalar


def _reference_run(steps, world, seed=0, lr=0.05):
    torch.manual_seed(seed)
    net = _Net()
    opt = torch.optim.AdamW(net.parameters(), lr=lr, weight_decay=0.01)
    losses = []
    for s in range(steps):
        total = 0.0
        opt.zero_grad()
        for r in range(world):                                   # the global batch is the union of the ranks' batches
            g = torch.Generator().manual_seed(100 * s + r)
            tok = torch.randint(0, 50, (2, 9), generator=g)
            loss = torch.nn.functional.cross_entropy(net(tok[:, :-1]).flatten(0, 1), tok[:, 1:].flatten(), reduction="sum")
            (loss / (world * 2 * 8)).backward()
            total += loss.item()
        opt.step()
        losses.append(total / (world * 2 * 8))
    return losses, {k: v.detach().clone() for k, v in net.state_dict().items()}


def _sharded_worker(rank, world, mode, steps, mixed):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    dist.init_process_group("gloo")
    from torchtitan_b200.parallel.fsdp import MixedPrecisionPolicy, fsdp_units, fully_shard, materialize, replicate

    torch.manual_seed(0)
    net = _Net()
    if mode == "hsdp":
        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("dp_replicate", "fsdp"))
    else:
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("fsdp",))
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16 if mixed else None, reduce_dtype=torch.float32)
    wrap = replicate if mode == "ddp" else fully_shard
    kw = {} if mode == "ddp" else {"reshard_after_forward": mode != "fsdp_noreshard"}
    if mode == "fsdp_offload":
        # shards "offloaded" with the CPU as compute device too: the same code path (separate master / gradient buffers,
        # compute copy refreshed from the master before every gather, gradients stored across the two), no device needed
        kw["compute_device"] = torch.device("cpu")
    for b in net.layers.values():
        wrap(b, mesh=mesh, mp_policy=mp, **kw)
    wrap(net, mesh=mesh, mp_policy=mp, **kw)
    materialize(net)
    params = [p for p in net.parameters()]
    opt = torch.optim.AdamW(params, lr=0.05, weight_decay=0.01)
    losses = []
    for s in range(steps):
        opt.zero_grad()
        g = torch.Generator().manual_seed(100 * s + rank)
        tok = torch.randint(0, 50, (2, 9), generator=g)
        logits = net(tok[:, :-1])
        loss = torch.nn.functional.cross_entropy(logits.float().flatten(0, 1), tok[:, 1:].flatten(), reduction="sum")
        (loss / (world * 2 * 8)).backward()
        for u in fsdp_units(net):
            u.wait_for_reduce()
        opt.step()
        for u in fsdp_units(net):
            u.mark_params_updated()
        t = torch.tensor([loss.item()])
        dist.all_reduce(t)
        losses.append(t.item() / (world * 2 * 8))
    # full parameters back: gather every sharded parameter
    full = {}
    for name, p in net.named_parameters():
        full[name] = p.full_tensor().detach().clone() if hasattr(p, "full_tensor") else p.detach().clone()
    shard_numel = sum((p._local_tensor if hasattr(p, "_local_tensor") else p).numel() for p in net.parameters())
    if mode == "fsdp_offload":
        assert all(u.offloaded and u.shadow_flat is not None and not any(u._slots) for u in fsdp_units(net))
    return {"losses": losses, "full": full, "shard_numel": shard_numel, "units": len(fsdp_units(net))}


@pytest.mark.parametrize("mode,world", [("fsdp", 2), ("fsdp_noreshard", 2), ("hsdp", 4), ("ddp", 2), ("fsdp", 3),
                                        ("fsdp_offload", 2)])
def test_sharded_training_matches_single_process(tmp_path, mode, world):
    steps = 4
    ref_losses, ref_state = _reference_run(steps, world)
    outs = run_ranks(_sharded_worker, world, mode, steps, False, tmp_path=tmp_path)
    for o in outs:
        assert o["losses"] == pytest.approx(ref_losses, rel=2e-5), (mode, o["losses"], ref_losses)
        for k, v in ref_state.items():
            assert torch.allclose(o["full"][k], v, rtol=2e-4, atol=2e-5), (mode, k)
        assert o["units"] == 4
    total = sum(v.numel() for v in ref_state.values())
    if mode.startswith("fsdp"):
        # every rank holds about 1 / world of the parameters (uneven rows are padded, the scalar is replicated)
        assert outs[0]["shard_numel"] < total / world * 1.25


def test_mixed_precision_shards_train_close_to_fp32(tmp_path):
    ref_losses, _ = _reference_run(4, 2)
    outs = run_ranks(_sharded_worker, 2, "fsdp", 4, True, tmp_path=tmp_path)
    assert outs[0]["losses"] == pytest.approx(ref_losses, rel=3e-2)      # bf16 compute copy, fp32 master and reduction


# ------------------------------------------------------------------------------------------ activation checkpointing
def _count_policy_decisions(mm_policy, force=()):
    """Run one block under per-op SAC and report (matmuls executed in forward, matmuls re-executed in backward)."""
    from torch.utils._python_dispatch import TorchDispatchMode

    from torchtitan_b200.config import ActivationCheckpointConfig
    from torchtitan_b200.parallel.ac import _apply_op_sac

    class Count(TorchDispatchMode):
        def __init__(self):
            super().__init__()
            self.n = 0

        def __torch_dispatch__(self, func, types, args=(), kwargs=None):
            if func == torch.ops.aten.mm.default:
                self.n += 1
            return func(*args, **(kwargs or {}))

    class Four(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b, self.c, self.d = (nn.Linear(16, 16, bias=False) for _ in range(4))

        def forward(self, x):
            return self.d(torch.relu(self.c(torch.relu(self.b(torch.relu(self.a(x)))))))

    torch.manual_seed(0)
    m = Four()
    ref = copy.deepcopy(m)
    cfg = ActivationCheckpointConfig(mode="selective", selective_ac_option="op", per_op_sac_mm_policy=mm_policy,
                                     per_op_sac_force_recompute_mm_shapes_by_fqns=list(force))
    _apply_op_sac(m, cfg, base_fqn="blk")
    x = torch.randn(6, 16, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    with Count() as fwd:
        y = m(x)
    with Count() as bwd:
        y.sum().backward()
    ref(xr).sum().backward()
    assert torch.allclose(x.grad, xr.grad, atol=1e-6)
    for p, q in zip(m.parameters(), ref.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6)
    # backward runs two gradient matmuls per linear (input and weight): 8; anything beyond is recomputation
    return fwd.n, bwd.n - 8


def test_per_op_sac_keeps_every_second_matmul_or_all():
    assert _count_policy_decisions("every_second") == (4, 2)        # two of four matmuls are recomputed
    assert _count_policy_decisions("all") == (4, 0)
    assert _count_policy_decisions("auto") == (4, 2)                # no CUDA device here: memory-bound choice


def test_full_and_layer_frequency_checkpointing_preserve_gradients():
    from torchtitan_b200.config import ActivationCheckpointConfig
    from torchtitan_b200.parallel import ac

    torch.manual_seed(0)
    net = _Net()
    ref = copy.deepcopy(net)
    ac._layer_sac_count = 0
    cfg = ActivationCheckpointConfig(mode="selective", selective_ac_option="2")
    wrapped = [ac._apply_ac_to_transformer_block(b, cfg) for b in net.layers.values()]
    assert [getattr(b, "_ac_recomputes_forward", False) for b in wrapped] == [False, True, False]
    net2 = copy.deepcopy(ref)
    for b in net2.layers.values():
        ac._apply_ac_to_transformer_block(b, ActivationCheckpointConfig(mode="full"))
    tok = torch.randint(0, 50, (2, 8))
    for m in (net, net2, ref):
        m(tok).square().mean().backward()
    for (n1, p1), (_, p2), (_, p3) in zip(net.named_parameters(), net2.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p1.grad, p3.grad, atol=1e-6), n1
        assert torch.allclose(p2.grad, p3.grad, atol=1e-6), n1
    with pytest.raises(ValueError):
        ac._apply_ac_to_transformer_block(net.layers["0"], ActivationCheckpointConfig(mode="selective", selective_ac_option="sometimes"))
    with pytest.raises(ValueError):
        ac._apply_ac_to_transformer_block(net.layers["0"], ActivationCheckpointConfig(mode="none"))


def _two_forwards_worker(rank, world):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    dist.init_process_group("gloo")
    from torchtitan_b200.config import ActivationCheckpointConfig
    from torchtitan_b200.parallel import ac
    from torchtitan_b200.parallel.fsdp import fsdp_units, fully_shard, materialize

    torch.manual_seed(0)
    net = _Net()
    ref = copy.deepcopy(net)
    for b in net.layers.values():
        ac._apply_ac_to_transformer_block(b, ActivationCheckpointConfig(mode="full"))
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("fsdp",))
    for b in net.layers.values():
        fully_shard(b, mesh=mesh, reshard_after_forward=False)
    fully_shard(net, mesh=mesh, reshard_after_forward=False)
    materialize(net)
    toks = [torch.randint(0, 50, (2, 8), generator=torch.Generator().manual_seed(10 * rank + i)) for i in range(2)]
    # the order of a pipeline warm-up: both micro-batches go forward before the first one goes backward
    outs = [net(t).square().mean() for t in toks]
    for o in outs:
        o.backward()
    for u in fsdp_units(net):
        u.wait_for_reduce()
    for t in toks:
        ref(t).square().mean().backward()
    worst = 0.0
    for (n, p), (_, q) in zip(net.named_parameters(), ref.named_parameters()):
        g = q.grad.clone()
        dist.all_reduce(g)                                        # FSDP sums over ranks
        got = p.grad.full_tensor() if hasattr(p.grad, "full_tensor") else p.grad
        worst = max(worst, (got - g).abs().max().item())
    return worst


def test_checkpointed_blocks_with_two_forwards_in_flight(tmp_path):
    """Pipeline schedules run several micro-batch forwards before the first backward; the recomputation of each
    micro-batch must see the parameter tensors of its own forward."""
    for worst in run_ranks(_two_forwards_worker, 2, tmp_path=tmp_path):
        assert worst < 1e-5, worst


def test_memory_budget_mixes_block_plans_and_preserves_gradients(tmp_path):
    """Reference: torchtitan/distributed/activation_checkpoint.py:216-230 hands the budget to the compiler's partitioner;
    here the same knob picks a per-block plan from a ladder (full / per-op / none)."""
    from torchtitan_b200.config import ActivationCheckpointConfig
    from torchtitan_b200.parallel import ac

    assert ac.plan_memory_budget(4, 0.0) == ["full"] * 4
    assert ac.plan_memory_budget(4, 1.0) == ["none"] * 4
    assert ac.plan_memory_budget(4, 0.22) == ["full", "op_every_second", "full", "op_every_second"]
    assert ac.plan_memory_budget(8, 0.5).count("op_all") == 3           # 0.40 + 3/8 * 0.25 <= 0.5
    shares = {n: m for n, m, _ in ac._BUDGET_LADDER}
    prev = -1.0
    for i in range(11):                                                   # monotone in the budget, never above it
        pl = ac.plan_memory_budget(6, i / 10)
        mean = sum(shares[x] for x in pl) / 6
        assert prev <= mean <= max(i / 10, shares["full"]) + 1e-9
        prev = mean
    with pytest.raises(ValueError):
        ac.plan_memory_budget(4, 1.5)

    torch.manual_seed(0)
    ref = _Net()
    tok = torch.randint(0, 50, (2, 8))
    ref(tok).square().mean().backward()
    for budget in (0.0, 0.3, 0.6, 1.0):
        net = copy.deepcopy(ref)
        net.zero_grad()
        ac.apply_ac(net, ActivationCheckpointConfig(mode="memory_budget", memory_budget=budget,
                                                    visualize_memory_budget_pareto=True), base_folder=str(tmp_path))
        net(tok).square().mean().backward()
        for (n1, p1), (_, p2) in zip(net.named_parameters(), ref.named_parameters()):
            assert torch.allclose(p1.grad, p2.grad, atol=1e-6), (budget, n1)
    rows = (tmp_path / "memory_budget_pareto.csv").read_text().strip().splitlines()
    assert rows[0] == "budget,resident_share,recompute_share" and len(rows) == 22


# ------------------------------------------------------------------------------------------ optimizer container
def test_optimizers_container_steps_and_round_trips_flattened_state():
    from torchtitan_b200.components.optimizer import OptimizersContainer

    class Second(nn.Module):                     # pipeline stages own disjoint parameter names
        def __init__(self):
            super().__init__()
            self.stage1 = _Net(n=1)

        def forward(self, tok):
            return self.stage1(tok)

    torch.manual_seed(0)
    a, b = _Net(n=1), Second()
    cfg = OptimizersContainer.Config(name="AdamW", lr=0.01, weight_decay=0.1, implementation="foreach")
    opt = OptimizersContainer(cfg, model_parts=[a, b])
    assert len(opt) == 2
    tok = torch.randint(0, 50, (2, 8))
    for m in (a, b):
        m(tok).square().mean().backward()
    before = a.out.weight.detach().clone()
    opt.step()
    opt.zero_grad()
    assert not torch.equal(before, a.out.weight) and a.out.weight.grad is None
    sd = opt.state_dict()
    assert any(k.startswith("state.") and k.endswith("exp_avg") for k in sd) and any("param_groups" in k for k in sd)
    a2, b2 = copy.deepcopy(a), copy.deepcopy(b)
    opt2 = OptimizersContainer(cfg, model_parts=[a2, b2])
    opt2.load_state_dict(copy.deepcopy(sd))      # a checkpoint read hands over fresh tensors, not the live state
    for m in (a, b, a2, b2):
        m(tok).square().mean().backward()
    opt.step()
    opt2.step()
    for p, q in zip(list(a.parameters()) + list(b.parameters()), list(a2.parameters()) + list(b2.parameters())):
        assert torch.equal(p, q)
    with pytest.raises(NotImplementedError):
        OptimizersContainer(OptimizersContainer.Config(name="Lion"), model_parts=[a])


def test_optimizers_in_backward_frees_gradients_as_it_goes():
    from torchtitan_b200.components.optimizer import OptimizersInBackwardContainer

    torch.manual_seed(0)
    net = _Net(n=1)
    ref = copy.deepcopy(net)
    cfg = OptimizersInBackwardContainer.Config(name="Adam", lr=0.01, weight_decay=0.0, implementation="for-loop")
    opt = OptimizersInBackwardContainer(cfg, model_parts=[net])
    ropt = torch.optim.Adam(ref.parameters(), lr=0.01)
    tok = torch.randint(0, 50, (2, 8))
    net(tok).square().mean().backward()          # the parameter hooks step and clear the gradients
    opt.step()
    opt.zero_grad()
    ref(tok).square().mean().backward()
    ropt.step()
    for p, q in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=1e-6)
        assert p.grad is None


def test_nvlink_staging_wait_is_needed_only_between_micro_batches_of_one_step():
    """The peer-memory transport waits for the peers' "read done" flags before a unit's next backward only when a
    reduce-scatter of that unit happened since the last optimizer step (host-side decision, no GPU needed)."""
    from types import SimpleNamespace

    from torchtitan_b200.parallel.nvlink_comm import NvlinkComm

    comm = NvlinkComm.__new__(NvlinkComm)
    unit = SimpleNamespace(params_version=3)
    comm._units = {}
    assert not comm.needs_staging_wait(unit)                       # unknown unit
    st = {"staging": object(), "grad_version": 0, "rs_params_version": None}
    comm._units[id(unit)] = st
    assert not comm.needs_staging_wait(unit)                       # nothing reduced yet
    st.update(grad_version=1, rs_params_version=3)
    assert comm.needs_staging_wait(unit)                           # second micro-batch of the same optimizer step
    unit.params_version = 4                                        # the optimizer ran: all-gather flags order the reuse
    assert not comm.needs_staging_wait(unit)


def _bucket_worker(rank, world, variant):
    """Llama debug model through ``apply_fsdp`` with the plan knobs of the graph trainer; returns losses and unit count."""
    import dataclasses
    from types import SimpleNamespace

    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.parallel import ParallelDims, fsdp
    from torchtitan_b200.parallel.data_parallel import apply_fsdp

    par = SimpleNamespace(fused_fsdp_collectives=False, fsdp_prefetch_depth=1, fsdp_bucket_bytes=0, fsdp_extra_process_group=False)
    for k, v in variant.items():
        setattr(par, k, v)
    pd = ParallelDims(dp_replicate=1, dp_shard=world, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=world)
    cfg = dataclasses.replace(llama3_configs["debugmodel"])
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=64)
    torch.manual_seed(5)
    model = cfg.build()
    model.init_weights()
    apply_fsdp(model, pd.get_mesh("fsdp"), param_dtype=torch.float32, reduce_dtype=torch.float32, pp_enabled=False,
               parallelism=par)
    fsdp.materialize(model)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(rank)
    losses = []
    for _ in range(3):
        x = torch.randint(0, cfg.vocab_size, (2, 65), generator=g)
        opt.zero_grad()
        loss = cross_entropy_loss(model(x[:, :-1]), x[:, 1:]) / (2 * 64 * world)
        loss.backward()
        opt.step()
        for u in fsdp.fsdp_units(model):
            u.mark_params_updated()
        l = loss.detach().clone()
        dist.all_reduce(l)
        losses.append(l.item())
    units = fsdp.fsdp_units(model)
    return losses, len(units), {u.prefetch_depth for u in units}


def test_bucketed_units_prefetch_depth_and_gather_group_keep_the_numbers(tmp_path):
    """What the graph trainer's plan sets on the FSDP runtime: grouping blocks into larger units, gathering two units
    ahead and a separate process group for all-gathers change the schedule, not the arithmetic."""
    for sub in "abc":
        (tmp_path / sub).mkdir()
    base = run_ranks(_bucket_worker, 2, {}, tmp_path=tmp_path / "a")[0]
    big = run_ranks(_bucket_worker, 2, {"fsdp_bucket_bytes": 1 << 30, "fsdp_prefetch_depth": 2}, tmp_path=tmp_path / "b")[0]
    pg = run_ranks(_bucket_worker, 2, {"fsdp_extra_process_group": True}, tmp_path=tmp_path / "c")[0]
    assert base[1] == 6 + 3 and big[1] == 1 + 3                  # 6 blocks -> one bucket; embedding, [norm, output], root stay
    assert base[2] == {1} and big[2] == {2}
    assert big[0] == pytest.approx(base[0], rel=1e-6) and pg[0] == pytest.approx(base[0], rel=1e-6)
    assert base[0][1] != base[0][0]                              # the optimizer steps in between did change the model


def _dtensor_worker(rank, world):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard

    dist.init_process_group("gloo")
    from torchtitan_b200.parallel.fsdp import dtensor_over

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("fsdp",))
    local = torch.arange(6, dtype=torch.float32).view(2, 3) + 10 * rank
    shape, stride = (2 * world, 3), (3, 1)
    kept = dtensor_over(local, mesh, [Shard(0)], shape, stride, keep_device=True)      # the path host-resident shards take
    moved = dtensor_over(local, mesh, [Shard(0)], shape, stride)
    same_storage = kept._local_tensor.data_ptr() == local.data_ptr()
    p = torch.nn.Parameter(kept)
    p.grad = dtensor_over(torch.ones(2, 3), mesh, [Shard(0)], shape, stride, keep_device=True)
    torch.optim.AdamW([p], lr=0.1, foreach=True).step()
    return {"equal": torch.equal(kept.full_tensor(), moved.full_tensor()), "same_storage": same_storage,
            "shape": tuple(kept.shape), "stepped": bool((p.to_local() != 10 * rank + torch.arange(6.0).view(2, 3)).any())}


def test_dtensor_built_from_its_spec_matches_from_local(tmp_path):
    """Host-resident shards under a device mesh of another type are wrapped without ``DTensor.from_local`` (which would
    move them): same global tensor, same storage, usable as a parameter with a gradient and an optimizer."""
    for o in run_ranks(_dtensor_worker, 2, tmp_path=tmp_path):
        assert o["equal"] and o["same_storage"] and o["shape"] == (4, 3) and o["stepped"]
