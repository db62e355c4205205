"""Metrics processor, distributed reductions, determinism seeds and gradient clipping over sharded parameters (gloo ranks on
CPU; model: the reference's tests/unit_tests/test_metrics? / distributed utils checks in test_utils and the clipping parity in
its FSDP integration tests)."""

import logging
import math

import pytest
import torch

from dist_utils import run_ranks


def _pd(world=1, **kw):
    from torchtitan_b200.parallel import ParallelDims

    base = dict(dp_replicate=1, dp_shard=world, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=world)
    base.update(kw)
    return ParallelDims(**base)


def test_metrics_processor_logs_throughput_and_writes_tensorboard(tmp_path, caplog):
    from torchtitan_b200.components.metrics import MetricsProcessor

    mp = MetricsProcessor(MetricsProcessor.Config(log_freq=5, enable_tensorboard=True, disable_color_printing=True),
                          parallel_dims=_pd(), dump_folder=str(tmp_path))
    assert mp.should_log(1) and mp.should_log(10) and not mp.should_log(7)
    with pytest.raises(AssertionError):
        mp.log(1, 1.0, 1.0, 0.5)                                # flops per token must be known first
    mp.num_flops_per_token = 6 * 1000
    mp.ntokens_since_last_log = 4096
    mp.data_loading_times.append(0.01)
    with caplog.at_level(logging.INFO):
        mp.log(5, 2.5, 2.75, 1.25, extra_metrics={"lr": 1e-3})
    text = " ".join(r.getMessage() for r in caplog.records)
    assert "step:  5" in text and "loss:  2.50000" in text and "grad_norm:  1.2500" in text and "tps:" in text and "mfu:" in text
    assert mp.ntokens_since_last_log == 0
    mp.close() if hasattr(mp, "close") else mp.logger.close()
    import glob

    assert glob.glob(str(tmp_path / "tb" / "*" / "events.out.tfevents.*"))


def test_metrics_reports_moe_load_histograms(tmp_path):
    from torchtitan_b200.components.metrics import MetricsProcessor

    class Block(torch.nn.Module):
        moe_enabled = True

        def __init__(self):
            super().__init__()
            self.moe = torch.nn.Module()
            self.moe.tokens_per_expert = torch.tensor([4.0, 0.0, 8.0, 4.0])

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleDict({"3": Block()})

    mp = MetricsProcessor(MetricsProcessor.Config(disable_color_printing=True), parallel_dims=_pd(), dump_folder=str(tmp_path))
    mp.model_parts = [M()]
    h = mp._moe_histograms()
    assert h["moe/layer_3/tokens_per_expert"] == [4.0, 0.0, 8.0, 4.0] and h["moe/layer_3/max_over_mean"] == 2.0


def _dist_worker(rank, world):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.config.configs import DebugConfig
    from torchtitan_b200.parallel import utils as dutils

    pd = _pd(world)
    mesh = pd.get_mesh("fsdp")
    x = torch.tensor(float(rank + 1))
    out = {
        "sum": dutils.dist_sum(x, mesh), "max": dutils.dist_max(x, mesh), "mean": dutils.dist_mean(x, mesh),
    }
    # seed: with no seed given rank 0's draw is broadcast, so all ranks agree
    dbg = DebugConfig(seed=None, deterministic=True)
    dutils.set_determinism(pd, torch.device("cpu"), dbg)
    out["draw"] = torch.rand(3)
    out["deterministic"] = torch.are_deterministic_algorithms_enabled()
    torch.use_deterministic_algorithms(False)
    return out


def test_distributed_reductions_and_shared_seed(tmp_path):
    outs = run_ranks(_dist_worker, 3, tmp_path=tmp_path)
    for o in outs:
        assert o["sum"] == 6.0 and o["max"] == 3.0 and o["mean"] == 2.0 and o["deterministic"]
        assert torch.equal(o["draw"], outs[0]["draw"])


def _clip_worker(rank, world, norm_type):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.parallel import fsdp
    from torchtitan_b200.parallel.utils import clip_grad_norm_

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.ReLU(), torch.nn.Linear(20, 7))
    ref = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.ReLU(), torch.nn.Linear(20, 7))
    ref.load_state_dict(net.state_dict())
    pd = _pd(world)
    fsdp.fully_shard(net, mesh=pd.get_mesh("fsdp"))
    fsdp.materialize(net)
    x = torch.randn(world, 5, 12)                                 # same data on every rank; rank r uses slice r
    net(x[rank]).square().sum().backward()
    for u in fsdp.fsdp_units(net):
        u.wait_for_reduce()
    ref(x.flatten(0, 1)).square().sum().backward()
    total = clip_grad_norm_(list(net.parameters()), 0.5, norm_type=norm_type)
    want = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5, norm_type=norm_type)
    g = net[2].weight.grad
    g = g.full_tensor() if hasattr(g, "full_tensor") else g
    return {"total": float(total), "want": float(want), "err": float((g - ref[2].weight.grad).abs().max())}


@pytest.mark.parametrize("norm_type", [2.0, math.inf, 1.0])
def test_clip_grad_norm_over_shards_matches_unsharded(tmp_path, norm_type):
    for o in run_ranks(_clip_worker, 2, norm_type, tmp_path=tmp_path):
        assert o["total"] == pytest.approx(o["want"], rel=1e-5)
        assert o["err"] < 1e-5


def test_seed_dtensor_rng_skips_cpu_meshes_and_forwards_cuda_ones(monkeypatch):
    """The DTensor tracker is created through ``manual_seed`` (no start-up broadcast over the default group)."""
    import types

    import torch.distributed.tensor._random as dtensor_random

    from torchtitan_b200.parallel import utils as dist_utils

    seen = []
    monkeypatch.setattr(dtensor_random, "manual_seed", lambda seed, mesh: seen.append((seed, mesh.device_type)))
    dist_utils.seed_dtensor_rng(None, 3)
    dist_utils.seed_dtensor_rng(types.SimpleNamespace(device_type="cpu"), 3)
    assert seen == []
    dist_utils.seed_dtensor_rng(types.SimpleNamespace(device_type="cuda"), 2**63 + 5)
    assert seen == [(5, "cuda")]


def test_trainer_raises_when_a_kernel_reports_an_expired_wait(monkeypatch):
    import types

    import torch

    from torchtitan_b200.ops import native
    from torchtitan_b200.trainer import Trainer

    fake = types.SimpleNamespace(device=torch.device("cuda"), step=7)
    fake._kernel_error_words = types.MethodType(Trainer._kernel_error_words, fake)
    monkeypatch.setattr(native, "available", lambda: True)
    monkeypatch.setattr(native, "kernel_errors", lambda: {})
    Trainer._raise_on_kernel_errors(fake)                         # nothing reported: no error
    monkeypatch.setattr(native, "kernel_errors", lambda: {"gemm": 4})
    with pytest.raises(RuntimeError, match="step 7.*gemm"):
        Trainer._raise_on_kernel_errors(fake)
    fake.device = torch.device("cpu")
    Trainer._raise_on_kernel_errors(fake)                         # CPU runs have no kernels to ask


def _fold_worker(rank, world):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.parallel import fsdp
    from torchtitan_b200.parallel.utils import clip_grad_norm_

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.ReLU(), torch.nn.Linear(20, 7))
    pd = _pd(world)
    fsdp.fully_shard(net[0], mesh=pd.get_mesh("fsdp"))
    fsdp.fully_shard(net, mesh=pd.get_mesh("fsdp"))
    fsdp.materialize(net)
    for p in net[0].parameters():                 # as for expert-parallel shards: the norm needs one more group
        p._extra_norm_groups = (dist.group.WORLD,)
    net(torch.randn(5, 12)).square().sum().backward()
    units = fsdp.fsdp_units(net)
    for u in units:
        u.wait_for_reduce()
    before = [u.grad_shard_flat.clone() for u in units]
    total = clip_grad_norm_(list(net.parameters()), 1e-3, fold_into_optimizer=True)
    coef = min(1.0, 1e-3 / (float(total) + 1e-6))
    return {"scales": [float(u.pending_grad_scale) for u in units], "coef": coef,
            "untouched": all(torch.equal(a, u.grad_shard_flat) for a, u in zip(before, units))}


def test_clip_coefficient_rides_into_the_flat_optimizer_for_every_unit(tmp_path):
    """With the clip folded into the flat-shard optimizer no gradient is scaled in place, also for units whose parameters
    carry extra norm groups (expert-parallel shards)."""
    for o in run_ranks(_fold_worker, 2, tmp_path=tmp_path):
        assert o["untouched"] and len(o["scales"]) == 2
        assert all(s == pytest.approx(o["coef"], rel=1e-5) for s in o["scales"])


def _node_worker(rank, world):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.parallel import nvlink_comm

    same = nvlink_comm.all_ranks_agree_on_one_node(dist.group.WORLD, True, "cpu")
    one_says_no = nvlink_comm.all_ranks_agree_on_one_node(dist.group.WORLD, rank != 1, "cpu")
    real = nvlink_comm.node_identity
    nvlink_comm.node_identity = lambda: real() ^ (rank == 2)         # rank 2 pretends to sit on another machine
    try:
        split = nvlink_comm.all_ranks_agree_on_one_node(dist.group.WORLD, True, "cpu")
    finally:
        nvlink_comm.node_identity = real
    no_gpu = nvlink_comm.peer_memory_group_ok(dist.group.WORLD)      # CPU ranks: never eligible, and nobody hangs
    return same, one_says_no, split, no_gpu


def test_peer_memory_groups_need_all_ranks_on_one_node(tmp_path):
    """CUDA IPC handles only mean something on the machine that made them: a group whose ranks report different node
    identities (a shard or tensor-parallel group that spans hosts in a multi-node job) must take the collectives, on
    every rank alike."""
    from torchtitan_b200.parallel.nvlink_comm import node_identity

    assert node_identity() == node_identity() and 0 <= node_identity() < 2**62
    for out in run_ranks(_node_worker, 3, tmp_path=tmp_path):
        assert out == (True, False, False, False)
