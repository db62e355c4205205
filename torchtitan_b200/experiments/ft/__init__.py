"""Replica-group fault tolerance: each replica group is its own launcher invocation; groups find each
other through a heartbeat/quorum service (native, ``csrc/ft/lighthouse.cpp``), average gradients over
the replicas that are alive at each step, and a group that rejoins pulls live state from a healthy one.
Counterpart of torchtitan/experiments/ft (which delegates these pieces to the external torchft package)."""

from .lighthouse import Lighthouse, LighthouseClient, Quorum
from .manager import FTManager, ReplicaManager

__all__ = ["Lighthouse", "LighthouseClient", "Quorum", "FTManager", "ReplicaManager", "has_torchft", "maybe_semi_sync_training"]

#: the reference gates its fault-tolerance code on the external torchft package; the quorum service, replica manager and
#: semi-synchronous methods of this framework are built in
has_torchft = True


def __getattr__(name):
    if name == "maybe_semi_sync_training":
        from .trainer import maybe_semi_sync_training

        return maybe_semi_sync_training
    raise AttributeError(name)
