"""Mixture-of-experts building blocks on CPU: router, reorderer, permute indices, expert-bias load balancing and the whole
layer against an explicit per-token loop (model: the reference's tests/unit_tests/test_moe? style checks of
models/common/moe and the kernels' CPU definition ``fill_indices_cpu``)."""

import pytest
import torch


def _router(**kw):
    from torchtitan_b200.models.common.moe.moe import TokenChoiceTopKRouter

    base = dict(dim=16, num_experts=8, num_expert_groups=None, num_limited_groups=None, top_k=2, score_func="softmax",
                route_norm=False, route_scale=1.0, gate_bias=False)
    base.update(kw)
    r = TokenChoiceTopKRouter(**base)
    torch.manual_seed(0)
    r.init_weights(init_std=0.5)
    return r


@pytest.mark.parametrize("score_func", ["softmax", "sigmoid"])
def test_router_picks_top_k_and_counts_tokens(score_func):
    r = _router(score_func=score_func)
    x = torch.randn(64, 16)
    top, idx, counts = r(x)
    logits = x @ r.gate.weight.t()
    scores = torch.softmax(logits, -1) if score_func == "softmax" else torch.sigmoid(logits)
    want = scores.topk(2, dim=-1)
    assert torch.equal(idx.sort(-1).values, want.indices.sort(-1).values)
    assert torch.allclose(top.sort(-1).values, want.values.sort(-1).values, atol=1e-6)
    assert counts.tolist() == torch.bincount(idx.flatten(), minlength=8).float().tolist() and counts.sum() == 128


def test_router_normalisation_scale_bias_and_groups():
    x = torch.randn(32, 16)
    top, _, _ = _router(route_norm=True, route_scale=2.5, score_func="sigmoid")(x)
    assert torch.allclose(top.sum(-1), torch.full((32,), 2.5), atol=1e-5)
    # the expert bias steers the choice but not the weights
    r = _router()
    bias = torch.zeros(8)
    bias[3] = 100.0
    top_b, idx_b, _ = r(x, bias)
    assert (idx_b == 3).any(-1).all()
    scores = torch.softmax(x @ r.gate.weight.t(), -1)
    assert torch.allclose(top_b.sort(-1).values, scores.gather(1, idx_b).sort(-1).values, atol=1e-6)
    # node-limited routing: experts come from at most `num_limited_groups` groups
    g = _router(num_expert_groups=4, num_limited_groups=1, top_k=2)
    _, idx_g, _ = g(x)
    assert ((idx_g // 2)[:, 0] == (idx_g // 2)[:, 1]).all()
    with pytest.raises(ValueError):
        _router(num_expert_groups=4, num_limited_groups=None)(x)
    with pytest.raises(ValueError):
        _router(num_expert_groups=3, num_limited_groups=1)(x)
    # forced balance: every expert gets the same number of pairs
    _, _, c = _router(_debug_force_load_balance=True)(x)
    assert c.tolist() == [8.0] * 8


def test_reorderer_is_a_stable_sort_by_expert():
    from torchtitan_b200.models.common.moe.moe import TokenReorderer

    idx = torch.tensor([[2, 0], [1, 2], [0, 1], [2, 1]])
    top = torch.arange(8, dtype=torch.float32).view(4, 2)
    scores, order, counts = TokenReorderer(num_experts=3, top_k=2)(top, idx)
    assert counts.tolist() == [2, 3, 3]
    assert order.tolist() == [1, 4, 2, 5, 7, 0, 3, 6]             # flat pair indices grouped by expert, original order kept
    assert scores.tolist() == [1.0, 4.0, 2.0, 5.0, 7.0, 0.0, 3.0, 6.0]


def test_permute_indices_regroup_by_local_expert_with_padding():
    from torchtitan_b200.models.common.moe.permute import generate_permute_indices

    # 2 ranks x 3 local experts; rows arrive ordered [rank][expert]
    counts = torch.tensor([2, 0, 3, 1, 4, 0], dtype=torch.int32)
    idx, sizes, offs = generate_permute_indices(counts, 3, 2, max_len=32, alignment=4)
    assert sizes.tolist() == [4, 4, 4] and offs.tolist() == [4, 8, 12]
    starts = (torch.cumsum(counts, 0) - counts).tolist()
    want = []
    for e in range(3):
        rows = []
        for r in range(2):
            i = r * 3 + e
            rows += list(range(starts[i], starts[i] + int(counts[i])))
        want += rows + [-1] * (4 - len(rows))
    assert idx[:12].tolist() == want and (idx[12:] == -1).all()
    # an empty expert still occupies one aligned block; a short output buffer truncates
    idx2, sizes2, _ = generate_permute_indices(torch.tensor([0, 5], dtype=torch.int32), 2, 1, max_len=10, alignment=8)
    assert sizes2.tolist() == [8, 8] and idx2.tolist() == [-1] * 8 + [0, 1]


def test_moe_layer_equals_per_token_loop():
    from torchtitan_b200.models.common.moe import MoE

    torch.manual_seed(0)
    moe = MoE.Config(num_experts=4, num_shared_experts=1, top_k=2, hidden_dim=24, score_func="sigmoid", route_norm=True,
                     score_before_experts=False).build(dim=12)
    moe.init_weights(init_std=0.3, buffer_device=torch.device("cpu"))
    x = torch.randn(2, 5, 12)
    y = moe(x)
    xt = x.reshape(-1, 12)
    top, idx, _ = moe.router(xt, moe.expert_bias)
    w1, w2, w3 = moe.experts.w1, moe.experts.w2, moe.experts.w3
    want = torch.zeros_like(xt)
    for t in range(xt.shape[0]):
        for s in range(2):
            e = int(idx[t, s])
            h = torch.nn.functional.silu(xt[t] @ w1[e].t()) * (xt[t] @ w3[e].t())
            want[t] += top[t, s] * (h @ w2[e].t())
    want = want + moe.shared_experts(xt)
    assert torch.allclose(y.reshape(-1, 12), want, atol=1e-5)
    assert moe.tokens_per_expert.sum() == 20
    # scores applied before the experts give a different (but finite) result with the same routing
    moe.score_before_experts = True
    y2 = moe(x)
    assert torch.isfinite(y2).all() and not torch.allclose(y2, y)


def test_expert_bias_update_moves_load_towards_balance():
    from torchtitan_b200.components.optimizer import OptimizersContainer, register_moe_load_balancing_hook
    from torchtitan_b200.models.common.moe import MoE
    from torchtitan_b200.parallel import ParallelDims

    class Block(torch.nn.Module):
        moe_enabled = True

        def __init__(self):
            super().__init__()
            self.moe = MoE.Config(num_experts=4, num_shared_experts=0, top_k=1, hidden_dim=8, load_balance_coeff=0.1).build(dim=8)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleDict({"0": Block()})

    net = Net()
    net.layers["0"].moe.init_weights(init_std=0.02, buffer_device=torch.device("cpu"))
    opt = OptimizersContainer(OptimizersContainer.Config(lr=0.0, implementation="for-loop"), model_parts=[net])
    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=1)
    register_moe_load_balancing_hook(opt, [net], pd)
    moe = net.layers["0"].moe
    moe.tokens_per_expert.copy_(torch.tensor([10.0, 2.0, 4.0, 0.0]))     # mean 4: expert 0 overloaded, 1 and 3 underloaded
    for p in net.parameters():
        p.grad = torch.zeros_like(p)
    opt.step()
    b = moe.expert_bias
    assert b[0] < 0 and b[1] > 0 and b[3] > 0 and abs(float(b.sum())) < 1e-6      # centred update of size coeff
    assert moe.tokens_per_expert.sum() == 0                                         # counters restart every step
