"""Fault tolerance on the host: the native heartbeat/quorum service, replica managers in separate CPU processes
(a replica that exits, one that goes silent, one that rejoins behind), commit voting, LocalSGD / DiLoCo."""

import multiprocessing as mp
import os
import time

import pytest
import torch


def _mk(lh, rid, **kw):
    from torchtitan_b200.experiments.ft import ReplicaManager

    return ReplicaManager(lighthouse_addr=lh, replica_id=rid, timeout_ms=4000, quorum_timeout_ms=8000, **kw)


def test_lighthouse_quorum_membership_and_silent_replica():
    from torchtitan_b200.experiments.ft import Lighthouse, LighthouseClient

    lh = Lighthouse(heartbeat_timeout_ms=600, join_timeout_ms=200)
    try:
        a, b = LighthouseClient(lh.address, "a", 50), LighthouseClient(lh.address, "b", 50)
        time.sleep(0.15)
        import threading

        res = {}
        t = threading.Thread(target=lambda: res.setdefault("b", b.quorum(7, 1, 3000, "h:2")))
        t.start()
        qa = a.quorum(5, 1, 3000, "h:1")
        t.join()
        assert qa.replica_ids == ["a", "b"] and res["b"].quorum_id == qa.quorum_id
        assert qa.max_step == 7 and qa.max_step_replica == "b" and qa.addresses == ["h:1", "h:2"]
        # b goes silent (no heartbeats, no quorum request): after the heartbeat timeout a forms a quorum alone
        b.pause_heartbeat(True)
        time.sleep(0.8)
        q2 = a.quorum(6, 1, 3000, "h:1")
        assert q2.replica_ids == ["a"] and q2.quorum_id == qa.quorum_id + 1
        # min_replicas cannot be met -> error reply, not a hang
        from torchtitan_b200.experiments.ft.lighthouse import QuorumError

        with pytest.raises(QuorumError, match="timeout"):
            a.quorum(7, 2, 400, "h:1")
        st = a.status()
        assert st["members"] == 2 and st["alive"] == 1 and st["quorums"] >= 2
        a.close()
        b.close()
    finally:
        lh.shutdown()


def _replica(lh_addr, rid, steps, die_after, start_delay, q):
    try:
        torch.manual_seed(0)
        w = torch.zeros(4)
        state = {"w": w}
        time.sleep(start_delay)                                  # a late joiner is unknown to the service until now
        m = _mk(lh_addr, rid, min_replica_size=1, state_dict=lambda: {"w": state["w"].clone()},
                load_state_dict=lambda s: state["w"].copy_(s["w"]))
        while m.client.status()["alive"] < 2:                    # start together with at least one peer
            time.sleep(0.05)
        log = []
        while m.step < steps:
            qm = m.start_quorum()
            g = torch.full((4,), float(int(rid[-1]) + 1))          # replica r contributes gradient r+1
            m.allreduce(g, average=True)
            if m.should_commit():
                state["w"] -= g
                log.append((m.step, len(qm.replica_ids), g[0].item()))
            time.sleep(0.15)
            if die_after is not None and m.step >= die_after:
                os._exit(0)                                         # a replica that disappears between steps
        q.put((rid, log, state["w"].tolist()))
        m.shutdown()
    except Exception as e:  # pragma: no cover
        import traceback

        q.put((rid, "ERR " + traceback.format_exc(), None))


def test_replicas_average_survive_a_death_and_heal_a_late_joiner():
    from torchtitan_b200.experiments.ft import Lighthouse

    lh = Lighthouse(heartbeat_timeout_ms=700, join_timeout_ms=6000)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    try:
        ps = [
            ctx.Process(target=_replica, args=(lh.address, "r0", 40, None, 0.0, q)),
            ctx.Process(target=_replica, args=(lh.address, "r1", 40, 3, 0.0, q)),     # exits after step 3
            ctx.Process(target=_replica, args=(lh.address, "r2", 40, None, 4.0, q)),  # joins late, must heal from r0
        ]
        for p in ps:
            p.start()
        out = {}
        for _ in range(2):
            rid, log, w = q.get(timeout=90)
            assert not isinstance(log, str), log
            out[rid] = (log, w)
        for p in ps:
            p.join(timeout=30)
        log0, w0 = out["r0"]
        log2, w2 = out["r2"]
        # while r0 and r1 were both alive the averaged gradient was (1 + 2) / 2
        assert any(n == 2 and g == 1.5 for _, n, g in log0)
        # after r1 died r0 kept committing (alone: g == 1, or with r2: (1 + 3) / 2 == 2)
        assert log0[-1][0] == 40 and any(g in (1.0, 2.0) for _, _, g in log0[4:])
        # the late joiner first took r0's state, so both end with identical weights
        assert w0 == w2, (w0, w2)
        assert log2[0][0] > 1   # it never replayed the steps it missed
    finally:
        lh.shutdown()


def _group_member(lh_addr, replica, rank, init_file, q):
    """One rank of a two-rank replica group (its own gloo group inside the replica, as a training job has)."""
    try:
        import torch.distributed as dist

        dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=2)
        m = _mk(lh_addr, f"g{replica}", min_replica_size=2, rank=rank, world_size=2)
        got = []
        for _ in range(3):
            qm = m.start_quorum()
            g = torch.full((2,), float((replica + 1) * 10 + rank))
            m.allreduce(g, average=True)
            if m.should_commit():
                got.append((len(qm.replica_ids), g[0].item()))
        q.put((replica, rank, got))
        m.shutdown()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback

        q.put((replica, rank, "ERR " + traceback.format_exc()))


def test_replica_groups_of_two_ranks_average_rank_by_rank(tmp_path):
    """Local rank r of every replica group forms its own cross-replica group (torchft's layout: the replicate dimension
    is managed per shard rank), all through one rendezvous store."""
    from torchtitan_b200.experiments.ft import Lighthouse

    lh = Lighthouse(heartbeat_timeout_ms=2000, join_timeout_ms=6000)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    try:
        ps = [ctx.Process(target=_group_member, args=(lh.address, rep, r, str(tmp_path / f"init{rep}"), q))
              for rep in range(2) for r in range(2)]
        for p in ps:
            p.start()
        res = [q.get(timeout=90) for _ in ps]
        for p in ps:
            p.join(timeout=30)
        for replica, rank, got in res:
            assert not isinstance(got, str), got
            assert got == [(2, 15.0 + rank)] * 3, (replica, rank, got)      # (10 + r + 20 + r) / 2
    finally:
        lh.shutdown()


class _FakeManager:
    """Two in-process 'replicas' averaged synchronously (no sockets): enough to test the semi-sync algebra."""

    def __init__(self, peers):
        self.peers, self.commit = peers, True

    def start_quorum(self):
        return None

    def allreduce(self, t, average=True):
        other = self.peers["other"](t)
        t.add_(other)
        if average:
            t.div_(2)
        return t

    def should_commit(self):
        return self.commit


def test_diloco_outer_step_and_uncommitted_sync():
    from torchtitan_b200.experiments.ft.local_sgd import DiLoCo

    torch.manual_seed(0)
    model = torch.nn.Linear(4, 4, bias=False)
    w_start = model.weight.detach().clone()
    inner = torch.optim.SGD(model.parameters(), lr=0.1)
    mgr = _FakeManager({"other": lambda t: torch.zeros_like(t)})   # the other replica did not move
    outer = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0, momentum=0.0, nesterov=False)
    with DiLoCo(mgr, [model], inner, outer_optimizer=outer, sync_every=2) as d:
        for _ in range(2):
            inner.zero_grad()
            model(torch.ones(1, 4)).sum().backward()
            inner.step()
    assert d.syncs == 1
    local_after_inner = w_start - 2 * 0.1 * torch.ones(4, 4)
    # pseudo-gradient averaged with a replica that stayed put = half of ours; outer lr 1 applies it to the global copy
    expect = w_start - (w_start - local_after_inner) / 2
    assert torch.allclose(model.weight, expect, atol=1e-6)
    # an uncommitted sync rolls the fragment back to the last agreed parameters
    mgr.commit = False
    with DiLoCo(mgr, [model], inner, outer_optimizer=outer, sync_every=1) as d2:
        agreed = model.weight.detach().clone()
        inner.zero_grad()
        model(torch.ones(1, 4)).sum().backward()
        inner.step()
    assert d2.syncs == 0 and torch.equal(model.weight, agreed)


def test_local_sgd_averages_parameters_every_n_steps():
    from torchtitan_b200.experiments.ft.local_sgd import LocalSGD

    model = torch.nn.Linear(2, 2, bias=False)
    torch.nn.init.ones_(model.weight)
    opt = torch.optim.SGD(model.parameters(), lr=1.0)
    mgr = _FakeManager({"other": lambda t: torch.zeros_like(t)})
    with LocalSGD(mgr, model, opt, sync_every=2):
        for i in range(3):
            opt.zero_grad()
            model.weight.grad = torch.zeros(2, 2)
            opt.step()
            if i == 0:
                assert torch.equal(model.weight, torch.ones(2, 2))
            if i == 1:
                assert torch.equal(model.weight, torch.full((2, 2), 0.5))


def test_ft_manager_config_surface_and_dp_remap():
    from torchtitan_b200.experiments.ft import FTManager, Lighthouse
    from torchtitan_b200.experiments.ft.config import FaultTolerance

    off = FTManager(FaultTolerance())
    assert not off.enabled and off.get_dp_info(4, 1) == (4, 1)
    lh = Lighthouse()
    try:
        on = FTManager(FaultTolerance(enable=True, replica_id=1, group_size=3, lighthouse=lh.address))
        assert on.enabled and on.get_dp_info(4, 1) == (12, 5) and on.loss_sync_pg is on.manager
        on.manager.shutdown()
        with pytest.raises(ValueError):
            FTManager(FaultTolerance(enable=True, process_group="mpi", lighthouse=lh.address))
    finally:
        lh.shutdown()
