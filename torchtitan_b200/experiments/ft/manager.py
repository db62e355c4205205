"""Replica manager: quorum per step, a process group rebuilt whenever membership changes, averaged
gradients over live replicas, commit voting, and live recovery of a lagging replica.

``FTManager`` keeps the configuration surface of torchtitan/experiments/ft/manager.py:37-153
(``enable, process_group, process_group_timeout_ms, replica_id, group_size, min_replica_size,
semi_sync_method``; ``get_dp_info`` remaps the dataloader's data-parallel degree/rank to
``dp_degree * group_size`` / ``dp_degree * replica_id + dp_rank``; ``maybe_set_all_reduce_hook``
averages FSDP shard gradients across replicas; ``loss_sync_pg``). :class:`ReplicaManager` is the
piece the reference takes from torchft (``ft.Manager`` + ``ManagedProcessGroup``).

Cross-replica groups are stand-alone ``ProcessGroupGloo`` / ``ProcessGroupNCCL`` objects built on a
TCP store hosted by the quorum's first replica; they exist beside the job's default process group.
A collective that fails or times out marks the step as *errored*: ``should_commit`` then returns False
on every replica of the quorum and the optimizer step is skipped.
"""

from __future__ import annotations

import io
import os
import socket
from dataclasses import dataclass
from datetime import timedelta

import torch
import torch.distributed as dist

from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.tools.logging import logger

from .lighthouse import LighthouseClient, Quorum, QuorumError


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class ReplicaManager:
    def __init__(self, *, lighthouse_addr: str, replica_id: str, min_replica_size: int = 1, backend: str = "gloo",
                 timeout_ms: int = 10000, quorum_timeout_ms: int = 30000, rank: int = 0, world_size: int = 1,
                 state_dict=None, load_state_dict=None, heartbeat_interval_ms: int = 100, host: str = "127.0.0.1"):
        self.replica_id, self.min_replica_size, self.backend = replica_id, min_replica_size, backend
        self.timeout = timedelta(milliseconds=timeout_ms)
        self.quorum_timeout_ms = quorum_timeout_ms
        self.rank, self.world_size, self.host = rank, world_size, host
        self._state_dict, self._load_state_dict = state_dict, load_state_dict
        # only local rank 0 of a replica group talks to the lighthouse; the result is broadcast inside the group
        self.client = LighthouseClient(lighthouse_addr, replica_id, heartbeat_interval_ms) if rank == 0 else None
        self.step = 0
        self.quorum: Quorum | None = None
        self.pg = None
        self._store = None
        self._store_port = _free_port() if rank == 0 else 0
        self._errored = False
        self._healing = False
        self._needs_fresh_group = False
        self.commits = 0

    # ---- membership -----------------------------------------------------------------------------------------
    def set_state_dict_fns(self, load_state_dict, state_dict) -> None:
        self._load_state_dict, self._state_dict = load_state_dict, state_dict

    def start_quorum(self) -> Quorum:
        """Call once per step before any cross-replica collective."""
        self._errored = False
        if self.rank == 0:
            try:
                fresh = "!" if (self._needs_fresh_group and self.quorum is None) else ""
                q = self.client.quorum(self.step, self.min_replica_size, self.quorum_timeout_ms,
                                       f"{self.host}:{self._store_port}{fresh}")
                self._needs_fresh_group = False
                box = [q]
            except QuorumError as e:
                box = [e]
        else:
            box = [None]
        if self.world_size > 1:
            dist.broadcast_object_list(box, src=0)
        if isinstance(box[0], Exception):
            raise box[0]
        q: Quorum = box[0]
        changed = self.quorum is None or q.quorum_id != self.quorum.quorum_id
        if changed:
            try:
                self._reconfigure(q)
            except Exception as e:       # peers that vanished while the group was being built
                self.report_error(e)
                self.pg = None
                self.quorum = q
                return q
        prev, self.quorum = self.quorum, q
        self._healing = q.max_step > self.step
        if (self._healing or changed) and len(q.replica_ids) > 1:
            self._recover(q)
        return q

    def _reconfigure(self, q: Quorum) -> None:
        n, me = len(q.replica_ids), q.rank_of(self.replica_id)
        host, port = q.addresses[0].rsplit(":", 1)
        # one rendezvous store for the whole quorum, hosted by rank 0 of the first replica; local rank r of every replica
        # meets its peers (rank r of the other replicas) under its own prefix and forms its own cross-replica group
        is_master = me == 0 and self.rank == 0
        port = int(port)
        if is_master and self._store is None:
            self._store = dist.TCPStore(host, port, is_master=True, wait_for_workers=False, timeout=self.timeout)
            store = self._store
        elif is_master:
            store = self._store
        else:
            store = dist.TCPStore(host, port, is_master=False, timeout=self.timeout)
        store = dist.PrefixStore(f"q{q.quorum_id}/r{self.rank}", store)
        if self.backend == "nccl":
            opts = dist.ProcessGroupNCCL.Options()
            opts._timeout = self.timeout
            self.pg = dist.ProcessGroupNCCL(store, me, n, opts)
        else:
            self.pg = dist.ProcessGroupGloo(store, me, n, self.timeout)
        logger.info(f"[ft] replica {self.replica_id}: quorum {q.quorum_id} with {q.replica_ids}")

    def _recover(self, q: Quorum) -> None:
        """Every member takes the state of the replica with the highest step (a no-op for up-to-date ones)."""
        src = q.rank_of(q.max_step_replica)
        me = q.rank_of(self.replica_id)
        try:
            if me == src:
                buf = io.BytesIO()
                torch.save({"step": self.step, "state": self._state_dict() if self._state_dict else None}, buf)
                payload = torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8)
                size = torch.tensor([payload.numel()], dtype=torch.int64)
            else:
                size = torch.zeros(1, dtype=torch.int64)
            self._bcast(size, src)
            if me != src:
                payload = torch.empty(int(size.item()), dtype=torch.uint8)
            self._bcast(payload, src)
            if me != src and self.step < q.max_step:
                obj = torch.load(io.BytesIO(payload.numpy().tobytes()), weights_only=False)
                if self._load_state_dict and obj["state"] is not None:
                    self._load_state_dict(obj["state"])
                logger.info(f"[ft] replica {self.replica_id}: recovered from {q.max_step_replica} (step {self.step} -> {obj['step']})")
                self.step = obj["step"]
        except Exception as e:  # a failed transfer makes this step uncommittable, not fatal
            self.report_error(e)

    def _bcast(self, t: torch.Tensor, src: int) -> None:
        opts = dist.BroadcastOptions()
        opts.rootRank = src
        self.pg.broadcast([t], opts).wait(self.timeout)

    # ---- collectives -------------------------------------------------------------------------------------------
    def num_participants(self) -> int:
        return len(self.quorum.replica_ids) if self.quorum else 1

    def allreduce(self, tensor: torch.Tensor, average: bool = True) -> torch.Tensor:
        """In-place sum (or mean) over live replicas; on failure the tensor is left as is and the step is marked errored."""
        if self.num_participants() == 1:
            return tensor
        if self.pg is None:
            self._errored = True          # the group could not be built this step
            return tensor
        try:
            staged = tensor if (self.backend == "nccl" or not tensor.is_cuda) else tensor.detach().cpu()
            opts = dist.AllreduceOptions()
            opts.reduceOp = dist.ReduceOp.SUM
            self.pg.allreduce([staged], opts).wait(self.timeout)
            if average:
                staged.div_(self.num_participants())
            if staged is not tensor:
                tensor.copy_(staged)
        except Exception as e:
            self.report_error(e)
        return tensor

    def report_error(self, e: Exception) -> None:
        logger.warning(f"[ft] replica {self.replica_id}: step {self.step} errored: {e}")
        self._errored = True

    def should_commit(self) -> bool:
        """True when no replica of the quorum saw an error this step (a vote over the group); advances the step."""
        ok = not self._errored
        if self.pg is None and self.num_participants() > 1:
            ok = False
        if self.pg is not None and self.num_participants() > 1:
            flag = torch.tensor([0.0 if ok else 1.0])
            try:
                opts = dist.AllreduceOptions()
                opts.reduceOp = dist.ReduceOp.SUM
                self.pg.allreduce([flag], opts).wait(self.timeout)
                ok = flag.item() == 0.0
            except Exception as e:
                logger.warning(f"[ft] commit vote failed: {e}")
                ok = False
        if self._errored or not ok:
            # a failed collective leaves the group in an unknown state: ask for a fresh quorum id and rebuild
            self.pg = None
            self.quorum = None
            self._needs_fresh_group = True
        if ok:
            self.step += 1
            self.commits += 1
            if self.client is not None:
                self.client.set_step(self.step)
        return ok

    def shutdown(self) -> None:
        if self.client is not None:
            self.client.close()
            self.client = None
        self.pg = None


class FTManager(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        enable: bool = False
        process_group: str = "gloo"
        process_group_timeout_ms: int = 10000
        replica_id: int = 0
        group_size: int = 0
        min_replica_size: int = 1
        semi_sync_method: str | None = None
        lighthouse: str = ""
        """``host:port`` of the quorum service; defaults to the ``TT_LIGHTHOUSE`` (or ``TORCHFT_LIGHTHOUSE``) variable."""

    def __init__(self, config: Config):
        self.config = config
        self._manager: ReplicaManager | None = None
        if not config.enable:
            return
        if config.process_group not in ("gloo", "nccl"):
            raise ValueError(f"Unsupported process group: {config.process_group}")
        addr = config.lighthouse or os.environ.get("TT_LIGHTHOUSE") or os.environ.get("TORCHFT_LIGHTHOUSE", "")
        if not addr:
            raise ValueError("fault tolerance needs a lighthouse address (--fault_tolerance.lighthouse or TT_LIGHTHOUSE)")
        addr = addr.replace("http://", "")
        self.use_async_quorum = config.semi_sync_method is None
        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
        self._manager = ReplicaManager(
            lighthouse_addr=addr, replica_id=f"torchtitan_ft_{config.replica_id}", min_replica_size=config.min_replica_size,
            backend=config.process_group, timeout_ms=config.process_group_timeout_ms, rank=rank, world_size=world,
        )
        self.group_size, self.replica_id = config.group_size, config.replica_id

    @property
    def enabled(self) -> bool:
        return self._manager is not None

    @property
    def manager(self) -> ReplicaManager:
        assert self._manager is not None
        return self._manager

    def get_dp_info(self, dp_degree: int, dp_rank: int) -> tuple[int, int]:
        if self.enabled:
            return dp_degree * self.group_size, dp_degree * self.replica_id + dp_rank
        return dp_degree, dp_rank

    def maybe_set_all_reduce_hook(self, model_parts: list[torch.nn.Module]) -> None:
        """Registers the FSDP units (or plain parameters) whose reduced gradients are averaged over live replicas.
        The averaging itself runs once per optimizer step (``average_gradients``), after the last micro-batch has
        been accumulated into the units' flat gradient shards -- one collective per unit, not per parameter."""
        self._grad_sources = []
        if not (self.enabled and self.use_async_quorum):
            return
        from torchtitan_b200.parallel import fsdp

        for part in model_parts:
            units = fsdp.fsdp_units(part)
            if units:
                self._grad_sources += [("unit", u) for u in units]
            else:
                self._grad_sources += [("param", p) for p in part.parameters() if p.requires_grad]

    def average_gradients(self) -> None:
        for kind, obj in getattr(self, "_grad_sources", []):
            if kind == "unit":
                obj.wait_for_reduce()
                self.manager.allreduce(obj.grad_shard_flat, average=True)
            elif obj.grad is not None:
                g = obj.grad.to_local() if hasattr(obj.grad, "to_local") else obj.grad
                self.manager.allreduce(g, average=True)

    @property
    def loss_sync_pg(self):
        return self.manager if (self.enabled and self.use_async_quorum) else None
