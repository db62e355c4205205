"""Context parallel: head-tail sharding and both ring methods against full attention on CPU ranks."""

import math

import pytest
import torch

from dist_utils import run_ranks
from torchtitan_b200.parallel.cp import headtail_indices


def test_headtail_indices_cover_and_balance():
    S, cp = 64, 4
    seen = torch.cat([headtail_indices(S, cp, r) for r in range(cp)])
    assert sorted(seen.tolist()) == list(range(S))
    # causal work (number of visible keys) is equal across ranks
    work = [int((headtail_indices(S, cp, r) + 1).sum()) for r in range(cp)]
    assert len(set(work)) == 1


def _worker(rank, world, method):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.ops import reference as ref
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.cp import RingAttention, cp_shard

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=world, tp=1, pp=1, ep=1, etp=1, world_size=world)
    mesh = pd.get_mesh("cp")
    torch.manual_seed(0)
    B, S, H, Hkv, D = 2, 32, 4, 2, 16
    q = torch.randn(B, S, H, D, requires_grad=True)
    k = torch.randn(B, S, Hkv, D, requires_grad=True)
    v = torch.randn(B, S, Hkv, D, requires_grad=True)
    do = torch.randn(B, S, H, D)
    full = ref.attention(q, k, v, causal=True)
    full.backward(do)
    ql, kl, vl, dol = cp_shard(mesh, (q.detach(), k.detach(), v.detach(), do), (1, 1, 1, 1))
    ql, kl, vl = ql.requires_grad_(), kl.requires_grad_(), vl.requires_grad_()
    ring = RingAttention(mesh, method)
    out = ring(ql, kl, vl)
    out.backward(dol)
    (want_o, want_dq, want_dk, want_dv) = cp_shard(mesh, (full.detach(), q.grad, k.grad, v.grad), (1, 1, 1, 1))
    return {
        "o": (out - want_o).abs().max().item(), "dq": (ql.grad - want_dq).abs().max().item(),
        "dk": (kl.grad - want_dk).abs().max().item(), "dv": (vl.grad - want_dv).abs().max().item(),
    }


@pytest.mark.parametrize("method", ["allgather", "alltoall"])
def test_ring_attention_matches_full(tmp_path, method):
    for o in run_ranks(_worker, 2, method, tmp_path=tmp_path):
        assert max(o.values()) < 1e-4, o
