"""MoE kernels on the GPU (router, counting sort, gather / combine) vs the PyTorch definitions."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("E,K,func,norm", [(128, 8, "softmax", True), (64, 6, "softmax", False), (256, 8, "sigmoid", True), (8, 2, "sigmoid", False)])
def test_router_forward_backward(E, K, func, norm):
    from torchtitan_b200.ops import cuda_ops, native
    from torchtitan_b200.ops import reference as ref

    native.lib()
    torch.manual_seed(0)
    T, D = 777, 256
    x = torch.randn(T, D, device="cuda").bfloat16().requires_grad_()
    gw = (torch.randn(E, D, device="cuda") * 0.1).requires_grad_()
    bias = torch.randn(E, device="cuda") * 0.01
    kw = dict(top_k=K, score_func=func, route_norm=norm, route_scale=2.5)
    top, idx, counts = cuda_ops.moe_route(x, gw, None, bias, **kw)
    g_expert = torch.randn(T, E, device="cuda")          # upstream gradient per (token, expert): slot order may differ
    top.backward(g_expert.gather(1, idx))
    x2, gw2 = x.detach().clone().requires_grad_(), gw.detach().clone().requires_grad_()
    rtop, ridx, rcounts = ref.moe_route(x2, gw2, None, bias, **kw)
    rtop.backward(g_expert.gather(1, ridx))
    # the same experts are chosen (order inside the k may differ); a near-tie at the k-th place may flip for a rare token
    same = (idx.sort(-1).values == ridx.sort(-1).values).all(-1)
    assert same.float().mean() > 0.99, same.float().mean()
    assert (counts - rcounts).abs().sum() <= 2 * (~same).sum()
    a = torch.zeros(T, E, device="cuda").scatter_(1, idx, top)
    b = torch.zeros(T, E, device="cuda").scatter_(1, ridx, rtop)
    assert (a - b)[same].abs().max() < 1e-5, (a - b)[same].abs().max()
    if bool(same.all()):
        assert (gw.grad - gw2.grad).abs().max() < 2e-3 * max(1.0, gw2.grad.abs().max().item()), (gw.grad - gw2.grad).abs().max()
        assert (x.grad.float() - x2.grad.float()).abs().max() < 2e-2 * max(1.0, x2.grad.float().abs().max().item())


def test_counting_sort_is_stable():
    from torchtitan_b200.ops import cuda_ops, native
    from torchtitan_b200.ops import reference as ref

    native.lib()
    torch.manual_seed(0)
    for T, K, E in ((4096, 8, 128), (1000, 3, 7), (5, 2, 16)):
        idx = torch.randint(0, E, (T, K), device="cuda")
        order, counts = cuda_ops.moe_sort(idx, E)
        rorder, rcounts = ref.moe_sort(idx, E)
        assert torch.equal(order, rorder) and torch.equal(counts, rcounts.to(counts.dtype))


def test_gather_and_combine_with_padding():
    from torchtitan_b200.ops import cuda_ops, native

    native.lib()
    torch.manual_seed(0)
    T, K, D, R = 300, 4, 256, 1536
    x = torch.randn(T, D, device="cuda").bfloat16().requires_grad_()
    perm = torch.randperm(R, device="cuda")[: T * K]
    pair = torch.full((R,), -1, dtype=torch.int64, device="cuda")
    pair[perm] = torch.arange(T * K, device="cuda")
    pos = perm.to(torch.int32)
    src = torch.where(pair >= 0, pair // K, pair).to(torch.int32)
    rows = cuda_ops.moe_gather_src(x, src, pos, K)
    want = torch.where((pair >= 0).view(-1, 1), x.detach()[(pair.clamp(min=0) // K)], torch.zeros((), device="cuda", dtype=x.dtype))
    assert torch.equal(rows, want)
    w = torch.rand(T, K, device="cuda").requires_grad_()
    rows_in = rows.detach().clone().requires_grad_()
    out = cuda_ops.moe_combine_pos(rows_in, pos, pair, w, T, K)
    g = torch.randn_like(out)
    out.backward(g)
    r32 = rows.detach().float()[pos.long()].view(T, K, D)
    ref = (w.detach().view(T, K, 1) * r32).sum(1)
    assert (out.float() - ref).abs().max() < 2e-2 * ref.abs().max()
    gw_ref = (r32 * g.float().view(T, 1, D)).sum(-1)
    assert (w.grad - gw_ref).abs().max() < 2e-2 * gw_ref.abs().max()
    grow_ref = torch.zeros(R, D, device="cuda")
    grow_ref[pos.long()] = (w.detach().view(T, K, 1) * g.float().view(T, 1, D)).reshape(T * K, D)
    assert (rows_in.grad.float() - grow_ref).abs().max() < 2e-2 * grow_ref.abs().max()
    # gather backward = unweighted sum of the k copies
    rows.backward(torch.ones_like(rows))
    assert torch.equal(x.grad, torch.full_like(x.grad, float(K)))
