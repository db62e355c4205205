"""Generation kernels on the GPU (KV write, paged decode attention, sampler) vs the PyTorch definitions in fp32."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


@pytest.mark.parametrize("H,Hkv", [(16, 8), (8, 8), (32, 4), (16, 2)])
def test_paged_decode_and_kv_write(H, Hkv):
    from torchtitan_b200.ops import cuda_ops, native
    from torchtitan_b200.ops import serving

    native.lib()
    torch.manual_seed(0)
    B, D, bs, nblocks = 5, 128, 16, 256
    lens = [1, 17, 128, 300, 513]
    kc = torch.zeros(nblocks, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    maxb = (max(lens) + bs - 1) // bs
    tables = torch.zeros(B, maxb, dtype=torch.int32, device="cuda")
    free = torch.randperm(nblocks).tolist()
    ks, vs = [], []
    for b, n in enumerate(lens):
        blks = [free.pop() for _ in range((n + bs - 1) // bs)]
        tables[b, : len(blks)] = torch.tensor(blks, dtype=torch.int32)
        k = torch.randn(n, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(n, Hkv, D, device="cuda").bfloat16()
        slots = torch.tensor([blks[t // bs] * bs + t % bs for t in range(n)], dtype=torch.int32, device="cuda")
        cuda_ops.kv_write(kc, vc, k, v, slots)
        ks.append(k)
        vs.append(v)
    # the scatter is exact
    b, n = 3, lens[3]
    blk0 = int(tables[b, 0])
    assert torch.equal(kc[blk0, :bs], ks[b][:bs]) and torch.equal(vc[blk0, :bs], vs[b][:bs])
    q = torch.randn(B, H, D, device="cuda").bfloat16()
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = cuda_ops.paged_decode(q, kc, vc, tables, ctx, D**-0.5)
    torch.cuda.synchronize()
    g = H // Hkv
    for b, n in enumerate(lens):
        kf, vf = ks[b].float().repeat_interleave(g, 1), vs[b].float().repeat_interleave(g, 1)   # [n, H, D]
        s = torch.einsum("hd,nhd->hn", q[b].float(), kf) * D**-0.5
        ref = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), vf)
        assert _rel(out[b], ref) < 2e-2, (b, _rel(out[b], ref))
    # and the dispatching wrapper takes the kernel
    out2 = serving.paged_attention_decode(q, kc, vc, tables, ctx, D**-0.5)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sampler_greedy_and_multinomial(dtype):
    from torchtitan_b200.ops import cuda_ops, native
    from torchtitan_b200.ops import serving

    native.lib()
    torch.manual_seed(0)
    B, V = 64, 151936
    logits = (torch.randn(B, V, device="cuda") * 2).to(dtype)
    u = torch.rand(B, device="cuda")
    tok, lp = cuda_ops.sample(logits, 0.0, u)
    lf = logits.float()
    assert torch.equal(tok, lf.argmax(-1))
    assert (lp - torch.log_softmax(lf, -1).gather(1, tok.view(-1, 1)).squeeze(1)).abs().max() < 1e-3
    # multinomial: the picked token is where the index-order CDF crosses u (allow rounding at the boundary)
    for temp in (1.0, 0.7):
        tok, lp = cuda_ops.sample(logits, temp, u)
        probs = torch.softmax(lf.double() / temp, -1)
        cdf = probs.cumsum(-1)
        hi = cdf.gather(1, tok.view(-1, 1)).squeeze(1)
        lo = hi - probs.gather(1, tok.view(-1, 1)).squeeze(1)
        target = u.double()
        assert ((target >= lo - 1e-4) & (target <= hi + 1e-4)).all()
        assert (lp - torch.log_softmax(lf, -1).gather(1, tok.view(-1, 1)).squeeze(1)).abs().max() < 1e-3
    # frequencies follow the distribution: a 4-token vocabulary sampled many times
    small = torch.tensor([[0.0, 1.0, 2.0, -1.0]], device="cuda").repeat(20000, 1)
    tok, _ = cuda_ops.sample(small, 1.0, torch.rand(20000, device="cuda"))
    freq = torch.bincount(tok, minlength=4).float() / 20000
    assert (freq - torch.softmax(small[0], -1)).abs().max() < 0.02
    t2, _ = serving.sample_top_p(logits, 1.0, 1.0, u)
    assert torch.equal(t2, cuda_ops.sample(logits, 1.0, u)[0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sampler_nucleus(dtype):
    """top-p sampling in the kernel (bisection on the logit key, no sort) vs the sorted definition: the token lies in
    the nucleus, sits where the index-order CDF over the nucleus crosses u, and frequencies follow the renormalised
    distribution."""
    from torchtitan_b200.ops import cuda_ops, native, serving

    if not native.has("tt_sample_top_p"):
        pytest.skip("library built without tt_sample_top_p")
    torch.manual_seed(0)
    B, V = 64, 151936
    logits = (torch.randn(B, V, device="cuda") * 3).to(dtype)
    u = torch.rand(B, device="cuda")
    lf = logits.float()
    for temp, top_p in ((1.0, 0.9), (0.7, 0.5), (1.0, 0.05)):
        tok, lp = cuda_ops.sample(logits, temp, u, top_p)
        probs = torch.softmax(lf.double() / temp, -1)
        # nucleus with slack on the cut: everything the strict definition keeps at top_p - eps must contain no outsider
        loose = serving.nucleus_mask(probs, min(1.0, top_p + 1e-4))
        assert loose.gather(1, tok.view(-1, 1)).all()
        keep = serving.nucleus_mask(probs, top_p)
        cdf = (probs * keep).cumsum(-1)
        total = cdf[:, -1]
        hi = cdf.gather(1, tok.view(-1, 1)).squeeze(1)
        lo = hi - (probs * keep).gather(1, tok.view(-1, 1)).squeeze(1)
        target = u.double() * total
        inside = (target >= lo - 2e-4) & (target <= hi + 2e-4)
        assert inside.float().mean() > 0.95, inside.float().mean()      # rows whose cut differs by one tie may shift
        assert (lp - torch.log_softmax(lf, -1).gather(1, tok.view(-1, 1)).squeeze(1)).abs().max() < 1e-3
    small = torch.tensor([[0.0, 1.0, 2.0, -1.0]], device="cuda").repeat(20000, 1)      # p = .087 .237 .644 .032
    tok, _ = cuda_ops.sample(small, 1.0, torch.rand(20000, device="cuda"), 0.8)          # nucleus = {2, 1}
    freq = torch.bincount(tok, minlength=4).float() / 20000
    p = torch.softmax(small[0], -1)
    want = torch.tensor([0.0, p[1] / (p[1] + p[2]), p[2] / (p[1] + p[2]), 0.0], device="cuda")
    assert (freq - want).abs().max() < 0.02, freq
    t2, _ = serving.sample_top_p(small[:8], 1.0, 0.8, torch.rand(8, device="cuda"))
    assert set(t2.tolist()) <= {1, 2}
