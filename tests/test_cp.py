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


def _masked_worker(rank, world, kind, balancer):
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
    docs = torch.tensor([[0] * 5 + [1] * 14 + [2] * 13, [0] * 20 + [1] * 12]) if "doc" in kind else None
    window = 7 if "window" in kind else None
    sinks = torch.randn(H, requires_grad=True) if "sinks" in kind else None
    full = ref.attention(q, k, v, causal=True, doc_ids=docs, window=window, sinks=sinks)
    full.backward(do)
    ql, kl, vl, dol = cp_shard(mesh, (q.detach(), k.detach(), v.detach(), do), (1, 1, 1, 1), balancer)
    ql, kl, vl = ql.requires_grad_(), kl.requires_grad_(), vl.requires_grad_()
    dl = cp_shard(mesh, (docs,), (1,), balancer)[0] if docs is not None else None
    sl = sinks.detach().clone().requires_grad_() if sinks is not None else None
    out = RingAttention(mesh, "allgather", balancer)(ql, kl, vl, doc_ids=dl, window=window, sinks=sl)
    out.backward(dol)
    want_o, want_dq, want_dk, want_dv = cp_shard(mesh, (full.detach(), q.grad, k.grad, v.grad), (1, 1, 1, 1), balancer)
    res = {"o": (out - want_o).abs().max().item(), "dq": (ql.grad - want_dq).abs().max().item(),
           "dk": (kl.grad - want_dk).abs().max().item(), "dv": (vl.grad - want_dv).abs().max().item()}
    if sinks is not None:      # each rank holds the sink gradient of its own queries: the sum over ranks is the full one
        g = sl.grad.clone()
        dist.all_reduce(g)
        res["dsinks"] = (g - sinks.grad).abs().max().item()
    try:
        RingAttention(mesh, "alltoall", balancer)(ql, kl, vl, window=3)
        res["ring_rejects_masks"] = 1.0
    except NotImplementedError:
        res["ring_rejects_masks"] = 0.0
    return res


@pytest.mark.parametrize("kind,balancer", [("doc", "headtail"), ("window", "headtail"), ("doc+window+sinks", "headtail"),
                                           ("doc+sinks", None)])
def test_context_parallel_with_masks_matches_full(tmp_path, kind, balancer):
    """Reference: torchtitan/distributed/context_parallel.py (flex-attention block masks under CP)."""
    for o in run_ranks(_masked_worker, 2, kind, balancer, tmp_path=tmp_path):
        assert max(o.values()) < 1e-4, o


def _model_worker(rank, world):
    import dataclasses
    import types

    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.cp import apply_cp_to_attention_module, prepare_context_parallel_input

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=world, tp=1, pp=1, ep=1, etp=1, world_size=world)
    cfg = dataclasses.replace(llama3_configs["debugmodel_flex_attn"], n_layers=2)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=64)
    torch.manual_seed(3)
    ref = cfg.build()
    ref.init_weights()
    model = cfg.build()
    model.load_state_dict(ref.state_dict())
    eos = 5
    x = torch.randint(6, cfg.vocab_size, (2, 65))
    x[0, 9] = x[0, 30] = x[1, 44] = eos                       # three document boundaries
    inp, lab = x[:, :-1], x[:, 1:]
    tok = types.SimpleNamespace(eos_id=eos)
    masks = ref.get_attention_masks(inp, tok)
    ref_loss = cross_entropy_loss(ref(inp, attention_masks=masks), lab)
    ref_loss.backward()

    mesh = pd.get_mesh("cp")
    apply_cp_to_attention_module([b.attention.inner_attention for b in model.layers.values()], mesh, "flex")
    li, ll, extra = prepare_context_parallel_input(inp, lab, {"attention_masks": model.get_attention_masks(inp, tok)}, mesh, "cpu")
    loss = cross_entropy_loss(model(li, **extra), ll)
    loss.backward()
    total = loss.detach().clone()
    dist.all_reduce(total)
    g = model.layers["0"].attention.wq.weight.grad.clone()
    dist.all_reduce(g)
    return {"loss": abs(total.item() - ref_loss.item()) / ref_loss.item(),
            "wq": (g - ref.layers["0"].attention.wq.weight.grad).abs().max().item()}


def test_model_with_document_masks_under_context_parallel(tmp_path):
    for o in run_ranks(_model_worker, 2, tmp_path=tmp_path):
        assert o["loss"] < 1e-5 and o["wq"] < 1e-4, o
