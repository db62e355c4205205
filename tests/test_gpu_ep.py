"""Expert-parallel token exchange over peer memory (``csrc/ep.cu``): the kernels with all "ranks" emulated on one GPU (launch
after launch, nothing waits on a later launch), and the dispatcher end to end on 2 GPUs against the all-to-all dispatcher."""

import ctypes

import pytest
import torch

from dist_utils import run_ranks

pytestmark = pytest.mark.gpu


def _ptrs(tensors):
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p)), arr


def test_ep_exchange_kernels_single_gpu_emulation():
    from torchtitan_b200.ops import native

    L = native.lib()
    if not native.has("tt_ep_push"):
        pytest.skip("library built without the expert-parallel exchange kernels")
    torch.manual_seed(0)
    W, E, k, T, D, align = 4, 8, 2, 48, 64, 8
    El, n = E // W, T * k
    cap = n * 2 + El * align
    st = torch.cuda.current_stream().cuda_stream
    xs = [torch.randn(T, D, device="cuda").bfloat16() for _ in range(W)]
    idx = [torch.randint(0, E, (T, k), device="cuda") for _ in range(W)]
    order = [torch.argsort(i.flatten(), stable=True) for i in idx]
    counts = [torch.bincount(i.flatten(), minlength=E) for i in idx]
    tables = [torch.zeros(W, E, dtype=torch.int32, device="cuda") for _ in range(W)]
    flags = [torch.zeros(W, dtype=torch.int32, device="cuda") for _ in range(W)]
    recv = [torch.full((cap, D), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    ret = [torch.full((n, D), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    arrive_f = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(W)]
    arrive_r = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(W)]
    tp, k1 = _ptrs(tables)
    fp, k2 = _ptrs(flags)
    for r in range(W):
        assert L.tt_ep_publish_counts(counts[r].data_ptr(), tp, fp, W, r, E, 1, st) == 0
    maps = []
    i32 = lambda m: torch.empty(m, dtype=torch.int32, device="cuda")
    for r in range(W):
        m = dict(dst_rank=i32(n), dst_row=i32(n), rev_rank=i32(cap), rev_row=i32(cap), offs=i32(El), info=i32(2))
        assert L.tt_ep_build_maps(tables[r].data_ptr(), flags[r].data_ptr(), W, r, E, align, n, cap, 1, m["dst_rank"].data_ptr(),
                                  m["dst_row"].data_ptr(), m["rev_rank"].data_ptr(), m["rev_row"].data_ptr(),
                                  m["offs"].data_ptr(), m["info"].data_ptr(), None, D, st) == 0
        maps.append(m)
    rp, k3 = _ptrs(recv)
    ap, k4 = _ptrs(arrive_f)
    ctas = L.tt_ep_push_ctas()
    for r in range(W):
        src = (order[r] // k).to(torch.int32)
        assert L.tt_ep_push(xs[r].data_ptr(), src.data_ptr(), n, maps[r]["dst_rank"].data_ptr(), maps[r]["dst_row"].data_ptr(),
                            rp, ap, W, D, cap, st) == 0
    for r in range(W):
        assert L.tt_ep_wait(arrive_f[r].data_ptr(), W * ctas, st) == 0
    torch.cuda.synchronize()
    assert not native.kernel_errors()
    # expected layout on rank d: local experts in order, each padded to `align`, sources in rank order inside a group
    for d in range(W):
        row, ends = 0, []
        for el in range(El):
            e = d * El + el
            for s in range(W):
                rows = xs[s][(order[s] // k)][idx[s].flatten()[order[s]] == e]
                got = recv[d][row : row + rows.shape[0]]
                assert torch.equal(got, rows), (d, el, s)
                assert (maps[d]["rev_rank"][row : row + rows.shape[0]] == s).all()
                row += rows.shape[0]
            pad = -row % align
            assert (maps[d]["rev_rank"][row : row + pad] == -1).all()
            row += pad
            ends.append(row)
        assert maps[d]["offs"].tolist() == ends and int(maps[d]["info"][0]) == row
    # the way back: every rank returns what it received, each source gets its rows in its own sorted order
    tp2, k5 = _ptrs(ret)
    ap2, k6 = _ptrs(arrive_r)
    for d in range(W):
        assert L.tt_ep_push(recv[d].data_ptr(), None, cap, maps[d]["rev_rank"].data_ptr(), maps[d]["rev_row"].data_ptr(),
                            tp2, ap2, W, D, n, st) == 0
    for r in range(W):
        assert L.tt_ep_wait(arrive_r[r].data_ptr(), W * ctas, st) == 0
    torch.cuda.synchronize()
    assert not native.kernel_errors()
    for s in range(W):
        assert torch.equal(ret[s], xs[s][order[s] // k])


def test_ep_wait_reports_missing_arrivals():
    """A wait on a counter that nothing bumps gives up after its limit and reports through the error word."""
    from torchtitan_b200.ops import native

    L = native.lib()
    if not native.has("tt_ep_push"):
        pytest.skip("library built without the expert-parallel exchange kernels")
    L.tt_ep_set_wait_ns(200_000_000)
    try:
        c = torch.zeros(1, dtype=torch.int32, device="cuda")
        assert L.tt_ep_wait(c.data_ptr(), 5, torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        err = native.kernel_errors()
        assert err.get("ep", (0,))[0] == 4 and err["ep"][2] == 5
        assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0      # the context is still healthy
    finally:
        L.tt_ep_set_wait_ns(20_000_000_000)


def _worker(rank, world, score_before=False):
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from torchtitan_b200.models.common.moe import MoE
    from torchtitan_b200.ops import native
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.ep import AllToAllDispatcher, _shard_experts
    from torchtitan_b200.parallel.nvlink_ep import NvlinkDispatcher

    pd = ParallelDims(dp_replicate=1, dp_shard=world, cp=1, tp=1, pp=1, ep=world, etp=1, world_size=world)
    ep_mesh = pd.get_mesh("ep")
    assert NvlinkDispatcher.available(ep_mesh)
    kw = dict(num_experts=8, num_shared_experts=1, score_func="softmax", route_norm=True, top_k=2, hidden_dim=128,
              score_before_experts=score_before)
    torch.manual_seed(0)
    base = MoE.Config(**kw).build(dim=128)
    base.init_weights(init_std=0.05, buffer_device=torch.device("cpu"))
    out = {"y": [], "dx": [], "dw1": [], "dgate": []}
    mods = []
    for which in ("a2a", "nvlink", "nvlink_small"):
        moe = MoE.Config(**kw).build(dim=128)
        moe.load_state_dict(base.state_dict())
        moe = moe.cuda().bfloat16()
        moe.router.gate.float()
        _shard_experts(moe.experts, ep_mesh)
        if which == "a2a":
            moe.experts.dispatcher = AllToAllDispatcher(ep_mesh, 8, alignment=64)
        else:
            moe.experts.dispatcher = NvlinkDispatcher(ep_mesh, 8, alignment=64)
            if which == "nvlink_small":
                # lossless mode with a receive buffer far too small for the traffic: every call must notice that on
                # the host and go through the collectives instead of dropping rows
                moe.experts.dispatcher.capacity_factor = 0.05
        mods.append(moe)
    for it in range(3):                                            # several calls: both buffer parities, counters keep counting
        x = torch.randn(2, 96, 128, generator=torch.Generator().manual_seed(100 * it + rank)).cuda().bfloat16()
        res = []
        for moe in mods:
            for p in moe.parameters():
                p.grad = None
            xi = x.clone().requires_grad_()
            y = moe(xi)
            y.float().square().sum().backward()
            res.append((y.detach().float(), xi.grad.float(), moe.experts.w1.grad.float(), moe.router.gate.weight.grad.float()))
        rel = lambda a, b: float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))
        for key, (a, b) in zip(out, zip(res[1], res[0])):
            out[key].append(rel(a, b))
        for key, (a, b) in zip(out, zip(res[2], res[0])):
            out[key].append(rel(a, b))
    torch.cuda.synchronize()
    out["errors"] = native.kernel_errors()
    out["fallbacks"] = (mods[1].experts.dispatcher.fallback_calls, mods[2].experts.dispatcher.fallback_calls)
    return out


@pytest.mark.parametrize("score_before", [False, True])
def test_nvlink_dispatcher_matches_all_to_all_two_gpus(tmp_path, score_before):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    for o in run_ranks(_worker, 2, score_before, tmp_path=tmp_path):
        assert not o["errors"], o
        # same rows reach the same experts: results agree to bf16 rounding of the combine order
        assert max(o["y"]) < 2e-2 and max(o["dx"]) < 3e-2 and max(o["dw1"]) < 3e-2 and max(o["dgate"]) < 3e-2, o
        assert o["fallbacks"][0] == 0 and o["fallbacks"][1] >= 3, o      # roomy buffer: never; tiny buffer: every forward
