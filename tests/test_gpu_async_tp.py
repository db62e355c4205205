"""Async tensor parallel on 2 GPUs: fused all-gather GEMM vs the collective path, and a TP=2 model step with
``enable_async_tensor_parallel`` (skipped with fewer than two GPUs)."""

import dataclasses

import pytest
import torch

from dist_utils import run_ranks

pytestmark = pytest.mark.gpu


def _need_two():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")


def _worker(rank, world):
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from torchtitan_b200.ops import native
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.async_tp import AsyncTP

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=world, pp=1, ep=1, etp=1, world_size=world)
    atp = AsyncTP.maybe_create(pd.get_mesh("tp"))
    assert atp is not None
    torch.manual_seed(0)
    S, K, N = 2048, 1024, 1536
    x_full = torch.randn(1, S, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16().requires_grad_()
    xl = x_full[:, rank * S // world : (rank + 1) * S // world].clone().requires_grad_()
    errs = []
    for it in range(3):                       # several calls: exercises the double buffer and the version flags
        xg, y = atp.ag_linear(xl * (it + 1), w)
        want = (x_full.float() * (it + 1)) @ w.float().t()
        errs.append(((y.float() - want).abs().max() / want.abs().max()).item())
        assert torch.equal(xg, x_full * (it + 1))
    g = torch.randn_like(y)
    dist.broadcast(g, src=0)
    y.backward(g)
    torch.cuda.synchronize()
    xr = x_full.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    ((xr * 3) @ wr.t()).backward(g.float())
    gx_ref = xr.grad[:, rank * S // world : (rank + 1) * S // world] * world   # every rank back-propagates the same g
    return {
        "fwd": max(errs), "gemm_err": native.lib().tt_gemm_error(),
        "gw": ((w.grad.float() - wr.grad).abs().max() / wr.grad.abs().max()).item(),
        "gx": ((xl.grad.float() - gx_ref).abs().max() / gx_ref.abs().max()).item(),
        "calls": atp.fused_calls,
    }


def _rs_worker(rank, world):
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from torchtitan_b200.ops import native
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.async_tp import AsyncTP

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=world, pp=1, ep=1, etp=1, world_size=world)
    atp = AsyncTP.maybe_create(pd.get_mesh("tp"))
    assert atp is not None
    torch.manual_seed(0)
    S, K, N = 2048, 1536, 1024
    h_full = torch.randn(1, S, K, device="cuda").bfloat16()
    w_full = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    ks = slice(rank * K // world, (rank + 1) * K // world)
    h = h_full[..., ks].clone().requires_grad_()
    w = w_full[:, ks].clone().requires_grad_()
    assert atp.rs_supported(h, w)
    rows = slice(rank * S // world, (rank + 1) * S // world)
    errs = []
    for it in range(4):                       # several calls: both staging buffers, counters keep counting
        y = atp.linear_rs(h * (it + 1), w)
        want = ((h_full.float() * (it + 1)) @ w_full.float().t())[:, rows]
        errs.append(((y.float() - want).abs().max() / want.abs().max()).item())
    g_full = torch.randn(1, S, N, device="cuda").bfloat16()
    dist.broadcast(g_full, src=0)
    y.backward(g_full[:, rows])
    torch.cuda.synchronize()
    hr = h_full.detach().float().requires_grad_()
    wr = w_full.detach().float().requires_grad_()
    ((hr * 4) @ wr.t()).backward(g_full.float())
    gh_ref, gw_ref = hr.grad[..., ks], wr.grad[:, ks]
    return {
        "fwd": max(errs), "gemm_err": native.lib().tt_gemm_error(),
        "gw": ((w.grad.float() - gw_ref).abs().max() / gw_ref.abs().max()).item(),
        "gh": ((h.grad.float() - gh_ref).abs().max() / gh_ref.abs().max()).item(),
    }


def test_fused_linear_reduce_scatter_two_gpus(tmp_path):
    _need_two()
    for o in run_ranks(_rs_worker, 2, tmp_path=tmp_path):
        assert o["gemm_err"] == 0, o
        assert o["fwd"] < 1e-2 and o["gw"] < 2e-2 and o["gh"] < 2e-2, o


def test_fused_allgather_linear_two_gpus(tmp_path):
    _need_two()
    for o in run_ranks(_worker, 2, tmp_path=tmp_path):
        assert o["gemm_err"] == 0 and o["calls"] >= 3, o          # three forward calls; the backward adds its own fused launch
        assert o["fwd"] < 1e-2 and o["gw"] < 2e-2 and o["gx"] < 2e-2, o


def _model_worker(rank, world):
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.tp import apply_tp_to_decoder, finalize_tp

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=world, pp=1, ep=1, etp=1, world_size=world)
    cfg = dataclasses.replace(llama3_configs["debugmodel_gqa"], n_layers=2)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=512)
    out = {}
    losses = []
    for async_tp in (False, True):
        torch.manual_seed(7)
        model = cfg.build().cuda().bfloat16()
        model.init_weights(buffer_device=torch.device("cuda"))
        apply_tp_to_decoder(model, pd.get_mesh("tp"), loss_parallel=True, async_tp=async_tp)
        finalize_tp(model)
        x = torch.randint(0, cfg.vocab_size, (1, 513), device="cuda", generator=torch.Generator("cuda").manual_seed(1))
        loss = cross_entropy_loss(model(x[:, :-1]), x[:, 1:]) / 512
        loss.backward()
        losses.append(loss.item())
        if async_tp:
            ff = model.layers["0"].feed_forward
            out["fused_calls"] = ff._async_tp.fused_calls
    out["losses"] = losses
    return out


def test_tp2_model_async_tp_matches_collectives(tmp_path):
    _need_two()
    for o in run_ranks(_model_worker, 2, tmp_path=tmp_path):
        assert o["fused_calls"] >= 2, o
        assert abs(o["losses"][0] - o["losses"][1]) < 2e-2, o
