"""Expert parallel dispatch/combine against the single-process MoE layer (2 CPU ranks)."""

import torch

from dist_utils import run_ranks


def _worker(rank, world, with_fsdp):
    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.models.common.moe import MoE
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.ep import AllToAllDispatcher, _shard_experts

    pd = ParallelDims(dp_replicate=1, dp_shard=world, cp=1, tp=1, pp=1, ep=world, etp=1, world_size=world)
    ep_mesh = pd.get_mesh("ep")
    kw = dict(num_experts=8, num_shared_experts=1, score_func="softmax", route_norm=True, top_k=2, hidden_dim=32,
              score_before_experts=False)
    torch.manual_seed(0)
    ref = MoE.Config(**kw).build(dim=16)
    ref.init_weights(init_std=0.02, buffer_device=torch.device("cpu"))
    state = {k: v.clone() for k, v in ref.state_dict().items()}
    moe = MoE.Config(**kw).build(dim=16)
    moe.load_state_dict(state)
    _shard_experts(moe.experts, ep_mesh)
    moe.experts.dispatcher = AllToAllDispatcher(ep_mesh, 8, alignment=8)
    # every rank has its own tokens; the reference processes the concatenation of all ranks' tokens
    xs = [torch.randn(2, 12, 16, generator=torch.Generator().manual_seed(10 + r)) for r in range(world)]
    x = xs[rank].clone().requires_grad_()
    y = moe(x)
    y.pow(2).sum().backward()
    xr = [t.clone().requires_grad_() for t in xs]
    yr = [ref(t) for t in xr]
    sum(t.pow(2).sum() for t in yr).backward()
    n = 8 // world
    return {
        "y": (y - yr[rank]).abs().max().item(),
        "dx": (x.grad - xr[rank].grad).abs().max().item(),
        "dw1": (moe.experts.w1.grad - ref.experts.w1.grad[rank * n : (rank + 1) * n]).abs().max().item(),
        "hist": (moe.tokens_per_expert - ref.tokens_per_expert).abs().max().item() if world == 1 else 0.0,
    }


def test_ep2_matches_single_process(tmp_path):
    for o in run_ranks(_worker, 2, False, tmp_path=tmp_path):
        assert max(o.values()) < 1e-5, o


def _model_worker(rank, world):
    import dataclasses

    import torch.distributed as dist

    dist.init_process_group("gloo")
    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.models.qwen3 import qwen3_configs
    from torchtitan_b200.parallel import ParallelDims, fsdp
    from torchtitan_b200.parallel import utils as dist_utils
    from torchtitan_b200.parallel.data_parallel import apply_fsdp
    from torchtitan_b200.parallel.ep import apply_moe_ep_tp
    from torchtitan_b200.parallel.tp import finalize_tp

    pd = ParallelDims(dp_replicate=1, dp_shard=world, cp=1, tp=1, pp=1, ep=world, etp=1, world_size=world)
    cfg = qwen3_configs["debugmodel_moe"]
    cfg = dataclasses.replace(cfg, n_layers=2) if dataclasses.is_dataclass(cfg) else cfg
    torch.manual_seed(3)
    ref = cfg.build()
    ref.init_weights()
    full = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    model = cfg.build()
    model.load_state_dict(full)
    apply_moe_ep_tp(model, pd, None)
    apply_fsdp(model, pd.get_mesh("fsdp"), param_dtype=torch.float32, reduce_dtype=torch.float32, pp_enabled=False,
               efsdp_mesh=pd.get_optional_mesh("efsdp"))
    fsdp.materialize(model)
    finalize_tp(model)
    xs = [torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(50 + r)) for r in range(world)]
    ntok = sum(x[:, 1:].numel() for x in xs)
    x = xs[rank]
    loss = cross_entropy_loss(model(x[:, :-1]), x[:, 1:]) / ntok
    loss.backward()
    ref_loss = sum(cross_entropy_loss(ref(t[:, :-1]), t[:, 1:]) for t in xs) / ntok
    ref_loss.backward()
    tot = loss.detach().clone()
    dist.all_reduce(tot)
    ref_norm = torch.nn.utils.get_total_norm([p.grad for p in ref.parameters() if p.grad is not None])
    norm = dist_utils.clip_grad_norm_(list(model.parameters()), 1e9, ep_enabled=True)
    return {"loss": tot.item(), "ref": ref_loss.item(), "norm": float(norm) if norm is not None else -1.0,
            "ref_norm": float(ref_norm)}


def test_ep2_fsdp_model_loss_and_grad_norm(tmp_path):
    for o in run_ranks(_model_worker, 2, tmp_path=tmp_path):
        assert abs(o["loss"] - o["ref"]) < 1e-5, o
        assert abs(o["norm"] - o["ref_norm"]) < 1e-4 * max(1.0, o["ref_norm"]), o
