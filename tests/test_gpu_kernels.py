"""Numerics of every CUDA kernel against a plain PyTorch fp32 definition of the same op."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from torchtitan_b200.ops import cuda_ops, native

    native.lib()
    return cuda_ops


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


def _close(a, b, rtol, atol_frac):
    """Per-element check: |a - b| <= atol + rtol * |b| with atol a fraction of the reference's RMS, so that errors on
    small-magnitude elements are seen too (a max-over-max ratio hides them)."""
    a, b = a.float(), b.float()
    atol = atol_frac * b.pow(2).mean().sqrt().item()
    bad = (a - b).abs() > atol + rtol * b.abs()
    return bad.float().mean().item()


@pytest.fixture(params=["fused", "split"])
def bwd_form(request):
    """Run a test once with the fused attention backward (default) and once with the deterministic two-kernel form."""
    from torchtitan_b200.ops import cuda_ops

    old = cuda_ops.ATTN_BWD_FUSED
    cuda_ops.ATTN_BWD_FUSED = request.param == "fused"
    yield request.param
    cuda_ops.ATTN_BWD_FUSED = old


def _no_kernel_errors():
    from torchtitan_b200.ops import native

    torch.cuda.synchronize()
    assert not native.kernel_errors()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 192), (384, 768, 1024), (200, 264, 136), (4096, 4096, 1024)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm(ops, M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    want = a.float() @ b.float().t()
    A = a.t().contiguous() if a_mn else a
    Bm = b.t().contiguous() if b_mn else b
    got = ops.gemm(A, Bm, a_mn, b_mn, False)
    got32 = ops.gemm(A, Bm, a_mn, b_mn, True)
    _no_kernel_errors()
    assert _rel(got32, want) < 2e-3, _rel(got32, want)
    assert _rel(got, want) < 1e-2, _rel(got, want)
    assert _close(got32, want, rtol=1e-3, atol_frac=1e-3) == 0.0      # per element, fp32 output
    assert _close(got, want, rtol=8e-3, atol_frac=4e-3) == 0.0        # per element, bf16 output (one rounding)


@pytest.mark.parametrize("pair", [0, 1])
def test_gemm_both_tile_kernels(ops, pair):
    from torchtitan_b200.ops import native

    native.lib().tt_gemm_set_pair(pair)
    try:
        torch.manual_seed(2)
        for (M, N, K) in [(512, 768, 320), (1000, 520, 264)]:
            a = torch.randn(M, K, device="cuda").bfloat16()
            b = torch.randn(N, K, device="cuda").bfloat16()
            want = a.float() @ b.float().t()
            for a_mn, b_mn in [(False, False), (False, True), (True, True)]:
                A = a.t().contiguous() if a_mn else a
                Bm = b.t().contiguous() if b_mn else b
                got = ops.gemm(A, Bm, a_mn, b_mn, True)
                _no_kernel_errors()
                assert _rel(got, want) < 2e-3, (M, N, K, a_mn, b_mn, _rel(got, want))
    finally:
        native.lib().tt_gemm_set_pair(1)


def test_gemm_accumulate_and_strided(ops):
    torch.manual_seed(1)
    a = torch.randn(256, 512, device="cuda").bfloat16()
    b = torch.randn(384, 512, device="cuda").bfloat16()
    big = torch.zeros(256, 1024, device="cuda", dtype=torch.float32)
    out = big[:, 128 : 128 + 384]
    ops.gemm_into(a, b, out)
    ops.gemm_into(a, b, out, accumulate=True)
    _no_kernel_errors()
    want = 2 * (a.float() @ b.float().t())
    assert _rel(out, want) < 2e-3
    assert big[:, :128].abs().max() == 0 and big[:, 512:].abs().max() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,D", [(64, 4096), (1000, 128), (33, 2048), (4096, 512), (16, 16384), (300, 2048), (1025, 4096)])
def test_rmsnorm(ops, dtype, rows, D):
    torch.manual_seed(0)
    x = torch.randn(rows, D, device="cuda", dtype=dtype, requires_grad=True)
    w = (torch.randn(D, device="cuda") * 0.1 + 1).to(dtype).requires_grad_()
    y = ops.rms_norm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel(y, yr) < tol
    assert _rel(x.grad, xr.grad) < tol
    assert _rel(w.grad, wr.grad) < (3e-2 if dtype == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("layout", ["interleaved", "half"])
@pytest.mark.parametrize("use_pos", [False, True])
def test_rope(ops, layout, use_pos):
    from torchtitan_b200.ops import reference as ref

    torch.manual_seed(0)
    B, S, H, D = 2, 96, 4, 128
    x = torch.randn(B, S, H, D, device="cuda").bfloat16().requires_grad_()
    ang = torch.randn(256, D // 2, device="cuda")
    table = torch.stack((ang.cos(), ang.sin()), -1).contiguous()
    pos = torch.randint(0, 256, (B, S), device="cuda") if use_pos else None
    y = ops.rope(x, table, pos, layout)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = ref.rope(xr, table, pos, layout)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2


def test_swiglu(ops):
    torch.manual_seed(0)
    g = torch.randn(300, 1024, device="cuda").bfloat16().requires_grad_()
    u = torch.randn(300, 1024, device="cuda").bfloat16().requires_grad_()
    y = ops.swiglu(g, u)
    d = torch.randn_like(y)
    y.backward(d)
    gr, ur = g.detach().float().requires_grad_(), u.detach().float().requires_grad_()
    yr = torch.nn.functional.silu(gr) * ur
    yr.backward(d.float())
    assert _rel(y, yr) < 1e-2 and _rel(g.grad, gr.grad) < 1.5e-2 and _rel(u.grad, ur.grad) < 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy_and_logprobs(ops, dtype):
    torch.manual_seed(0)
    rows, V = 257, 4104
    logits = (torch.randn(rows, V, device="cuda") * 3).to(dtype).requires_grad_()
    labels = torch.randint(0, V, (rows,), device="cuda")
    labels[::7] = -100
    loss = ops.cross_entropy_sum(logits, labels, -100)
    (loss * 0.37).backward()
    lr = logits.detach().float().requires_grad_()
    want = torch.nn.functional.cross_entropy(lr, labels, reduction="sum", ignore_index=-100)
    (want * 0.37).backward()
    assert abs(loss.item() - want.item()) / want.item() < 1e-4
    assert _rel(logits.grad, lr.grad) < (2e-2 if dtype == torch.bfloat16 else 1e-4)
    # log-probs
    labels2 = torch.randint(0, V, (rows,), device="cuda")
    l2 = logits.detach().clone().requires_grad_()
    lp = ops.token_logprobs(l2, labels2)
    w = torch.randn(rows, device="cuda")
    (lp * w).sum().backward()
    l3 = logits.detach().float().requires_grad_()
    lpr = torch.log_softmax(l3, -1).gather(-1, labels2[:, None]).squeeze(-1)
    (lpr * w).sum().backward()
    assert (lp - lpr).abs().max() < 1e-3
    assert _rel(l2.grad, l3.grad) < (2e-2 if dtype == torch.bfloat16 else 1e-4)


def test_adamw_and_sumsq(ops):
    torch.manual_seed(0)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda") * 0.1
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    shadow = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        ops.adamw_flat(p, g, m, v, shadow, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        ref_p.grad = g.clone()
        opt.step()
    assert (p - ref_p.detach()).abs().max() < 1e-5
    assert (shadow.float() - p).abs().max() < 2e-2
    s = ops.sumsq(g)
    assert abs(s.item() - g.double().pow(2).sum().item()) / s.item() < 1e-5


@pytest.mark.parametrize("B,S,H,Hkv", [(1, 128, 2, 2), (2, 256, 4, 2), (1, 1024, 8, 2), (1, 384, 4, 1), (1, 2048, 4, 1)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention(ops, B, S, H, Hkv, causal, bwd_form):
    from torchtitan_b200.ops import reference as ref

    torch.manual_seed(0)
    D = 128
    q = torch.randn(B, S, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    assert ops.attention_supported(q, k)
    o, lse = ops.attention(q, k, v, causal=causal, return_lse=True)
    do = torch.randn_like(o)
    o.backward(do)
    _no_kernel_errors()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    g = H // Hkv
    s = torch.einsum("bqhd,bkhd->bhqk", qr, kr.repeat_interleave(g, 2)) / math.sqrt(D)
    if causal:
        s = s.masked_fill(torch.ones(S, S, device="cuda", dtype=torch.bool).triu(1), float("-inf"))
    lser = torch.logsumexp(s, -1)
    orf = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vr.repeat_interleave(g, 2))
    orf.backward(do.float())
    assert _rel(o, orf) < 2e-2, _rel(o, orf)
    assert (lse - lser).abs().max() < 2e-2
    assert _rel(q.grad, qr.grad) < 3e-2, _rel(q.grad, qr.grad)
    assert _rel(k.grad, kr.grad) < 3e-2, _rel(k.grad, kr.grad)
    assert _rel(v.grad, vr.grad) < 3e-2, _rel(v.grad, vr.grad)
    # per element: bf16 outputs of fp32-accumulated sums are within a few bf16 ulps (2^-8) of the fp32 result
    for got, want in ((o, orf), (q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert _close(got, want, rtol=2e-2, atol_frac=2e-2) < 1e-4


@pytest.mark.parametrize("kind", ["docs", "window", "docs+window", "block"])
@pytest.mark.parametrize("B,S,H,Hkv", [(2, 512, 4, 2), (1, 1024, 4, 1)])
def test_attention_range_masks(ops, kind, B, S, H, Hkv, bwd_form):
    """Document / sliding-window / fixed-block causal masks through the flash kernel vs an fp32 masked reference."""
    from torchtitan_b200.ops import reference as ref

    torch.manual_seed(1)
    D = 128
    q = torch.randn(B, S, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    doc, window = None, None
    if "docs" in kind:
        # boundaries that fall inside tiles, on tile edges and make very short documents
        cuts = torch.tensor([0, 5, 64, 130, 131, 300, 448][: 4 + S // 256], device="cuda")
        doc = (torch.arange(S, device="cuda").view(1, S) >= cuts.view(-1, 1)).sum(0, keepdim=True).int().expand(B, S).contiguous()
        if B > 1:
            doc = doc.clone()
            doc[1] = (torch.arange(S, device="cuda") // 200).int()
    if "window" in kind:
        window = 100
    if kind == "block":
        doc = (torch.arange(S, device="cuda") // 192).int().view(1, S).expand(B, S).contiguous()
    o, lse = ops.attention(q, k, v, causal=True, window=window, doc_ids=doc, return_lse=True)
    do = torch.randn_like(o)
    o.backward(do)
    _no_kernel_errors()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf, lser = ref.attention(qr, kr, vr, causal=True, window=window, doc_ids=doc, return_lse=True)
    orf.backward(do.float())
    assert _rel(o, orf) < 2e-2, _rel(o, orf)
    assert (lse - lser).abs().max() < 2e-2
    assert _rel(q.grad, qr.grad) < 3e-2, _rel(q.grad, qr.grad)
    assert _rel(k.grad, kr.grad) < 3e-2, _rel(k.grad, kr.grad)
    assert _rel(v.grad, vr.grad) < 3e-2, _rel(v.grad, vr.grad)


@pytest.mark.parametrize("window", [None, 128])
def test_attention_sinks(ops, window):
    """Per-head attention sinks (a logit in the softmax denominator that carries no value), with and without a sliding
    window, through the flash kernel vs the fp32 definition; the sink gradient comes from lse."""
    from torchtitan_b200.ops import reference as ref

    torch.manual_seed(2)
    B, S, H, Hkv, D = 2, 512, 8, 2, 128
    q = torch.randn(B, S, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    sinks = (torch.randn(H, device="cuda") * 2).requires_grad_()       # some above, some below the typical row maximum
    o, lse = ops.attention(q, k, v, causal=True, window=window, sinks=sinks, return_lse=True)
    do = torch.randn_like(o)
    o.backward(do)
    _no_kernel_errors()
    qr, kr, vr, sr = (t.detach().float().requires_grad_() for t in (q, k, v, sinks))
    orf, lser = ref.attention(qr, kr, vr, causal=True, window=window, sinks=sr, return_lse=True)
    orf.backward(do.float())
    assert _rel(o, orf) < 2e-2, _rel(o, orf)
    assert (lse - lser).abs().max() < 2e-2
    assert _rel(q.grad, qr.grad) < 3e-2, _rel(q.grad, qr.grad)
    assert _rel(k.grad, kr.grad) < 3e-2, _rel(k.grad, kr.grad)
    assert _rel(v.grad, vr.grad) < 3e-2, _rel(v.grad, vr.grad)
    assert _rel(sinks.grad, sr.grad) < 3e-2, _rel(sinks.grad, sr.grad)


@pytest.mark.parametrize("E,N,K,sizes", [
    (4, 256, 128, [64, 0, 192, 128]),
    (8, 768, 2048, [640, 64, 0, 128, 1024, 64, 320, 192]),
    (3, 192, 320, [128, 64, 64]),
    (2, 512, 256, [448, 832]),
])
@pytest.mark.parametrize("pair", [True, False])
def test_grouped_gemm_device_offsets(ops, E, N, K, sizes, pair):
    """Grouped GEMM with device-side group offsets (forward, input gradient, weight gradient) vs fp32 per-expert matmuls;
    256-row tiles on CTA pairs where the shape allows it, and the single-CTA kernel alone."""
    from torchtitan_b200.ops import native

    if native.has("tt_grouped_gemm_set_pair"):
        native.lib().tt_grouped_gemm_set_pair(int(pair))
    elif pair:
        pytest.skip("library built without the CTA-pair grouped GEMM")
    torch.manual_seed(0)
    R = sum(sizes) + 64                      # trailing padding rows belong to no group
    x = (torch.randn(R, K, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(E, N, K, device="cuda") * 0.05).bfloat16().requires_grad_()
    counts = torch.tensor(sizes, device="cuda", dtype=torch.int64)
    counts._tt_aligned = 64
    y = ops.grouped_linear(x, w, counts)
    gy = torch.randn_like(y)
    y.backward(gy)
    _no_kernel_errors()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    outs, s = [], 0
    for e, n in enumerate(sizes):
        outs.append(xr[s : s + n] @ wr[e].t())
        s += n
    outs.append(xr.new_zeros(R - s, N))
    yr = torch.cat(outs)
    yr.backward(gy.float())
    assert _rel(y, yr) < 2e-2, _rel(y, yr)
    assert (y[s:] == 0).all()
    assert _rel(x.grad, xr.grad) < 2e-2, _rel(x.grad, xr.grad)
    assert _rel(w.grad, wr.grad) < 2e-2, _rel(w.grad, wr.grad)
    if native.has("tt_grouped_gemm_set_pair"):
        native.lib().tt_grouped_gemm_set_pair(1)


def test_moe_layer_native_grouped_path(ops):
    """A MoE layer on the GPU (padded dispatcher + device-offset grouped GEMMs) vs the same layer in fp32 on the CPU."""
    from torchtitan_b200.models.common.moe import MoE

    kw = dict(num_experts=8, num_shared_experts=1, score_func="softmax", route_norm=True, top_k=2, hidden_dim=128,
              score_before_experts=False)
    torch.manual_seed(0)
    ref_moe = MoE.Config(**kw).build(dim=128)
    ref_moe.init_weights(init_std=0.02, buffer_device=torch.device("cpu"))
    moe = MoE.Config(**kw).build(dim=128)
    moe.load_state_dict(ref_moe.state_dict())
    moe = moe.cuda().bfloat16()
    moe.router.gate.float()
    x = torch.randn(2, 256, 128)
    xg = x.cuda().bfloat16().requires_grad_()
    xr = x.bfloat16().float().requires_grad_()
    y = moe(xg)
    y.float().square().sum().backward()
    _no_kernel_errors()
    yr = ref_moe(xr)
    yr.square().sum().backward()
    # a token whose two best scores are nearly tied may be routed differently by the two gate products: compare the
    # tokens on whose experts both sides agree (nearly all of them)
    with torch.no_grad():
        _, idx_g, _ = moe.router(xg.detach().reshape(-1, 128), moe.expert_bias)
        _, idx_r, _ = ref_moe.router(xr.detach().reshape(-1, 128), ref_moe.expert_bias)
    same = (idx_g.cpu().sort(-1).values == idx_r.sort(-1).values).all(-1)
    assert same.float().mean() > 0.98, same.float().mean()
    yg, yc = y.detach().cpu().reshape(-1, 128)[same], yr.detach().reshape(-1, 128)[same]
    assert _rel(yg, yc) < 5e-2, _rel(yg, yc)
    gg, gc = xg.grad.cpu().reshape(-1, 128)[same], xr.grad.reshape(-1, 128)[same]
    assert _rel(gg, gc) < 8e-2, _rel(gg, gc)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (512, 768, 1024), (300, 264, 208), (4096, 4096, 2048)])
@pytest.mark.parametrize("mode", ["tensorwise", "rowwise"])
def test_gemm_fp8(ops, M, N, K, mode):
    """tcgen05 float8 GEMM with epilogue scales vs the fp32 product of the dequantised operands."""
    from torchtitan_b200.ops import quant

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda") * 2
    b = torch.randn(N, K, device="cuda") * 0.3
    axis = None if mode == "tensorwise" else -1
    qa, sa = quant.quantize_fp8(a, axis)
    qb, sb = quant.quantize_fp8(b, axis)
    got = ops.gemm_fp8(qa, qb, sa, sb, torch.float32)
    _no_kernel_errors()
    want = (qa.float() * sa) @ (qb.float() * sb).t()
    assert _rel(got, want) < 1e-3, _rel(got, want)
    got16 = ops.gemm_fp8(qa, qb, sa, sb, torch.bfloat16)
    assert _rel(got16, want) < 1e-2
    # e5m2 gradients against e4m3 weights
    qg, sg = quant.quantize_fp8(a, None, torch.float8_e5m2)
    got = ops.gemm_fp8(qg, qb, sg, sb if mode == "tensorwise" else sb.mean(), torch.float32)
    want = (qg.float() * sg) @ (qb.float() * (sb if mode == "tensorwise" else sb.mean())).t()
    assert _rel(got, want) < 1e-3, _rel(got, want)


def test_smoke_step():
    from torchtitan_b200.tools.smoke import run_smoke

    loss = run_smoke()
    assert 0 < loss < 12


@pytest.mark.parametrize("rowwise", [True, False])
@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_fp8_quantise_kernels(ops, rowwise, dtype):
    """Native float8 quantisation of a GEMM operand (as stored, and as a transposed view) vs the elementwise definition:
    same scales, same 8-bit codes up to rounding of values that sit on a tie."""
    from torchtitan_b200.ops import cuda_ops
    from torchtitan_b200.ops.quant import quantize_fp8

    torch.manual_seed(0)
    for R, K in [(384, 1024), (272, 336)]:
        base = (torch.randn(R, K, device="cuda") * torch.rand(R, 1, device="cuda") * 8).bfloat16()
        base[3] = 0                                                    # an all-zero row takes the amax floor
        for x in (base, (torch.randn(K, R, device="cuda") * 3).bfloat16().t()):
            got = cuda_ops.quantize_fp8_operand(x, rowwise, dtype)
            assert got is not None
            q, scale = got
            qr, sr = quantize_fp8(x, -1 if rowwise else None, dtype)
            assert q.is_contiguous() and q.shape == x.shape and q.dtype == dtype
            if rowwise:
                assert torch.equal(scale.reshape(-1), sr.reshape(-1).float()), (scale.reshape(-1)[:4], sr.reshape(-1)[:4])
            else:
                # amax / fmax is a true division in the kernel and a multiplication by the reciprocal in the elementwise
                # definition on this device: one unit in the last place apart at most; codes are compared at the kernel's scale
                assert torch.allclose(scale.reshape(-1), sr.reshape(-1).float(), rtol=3e-7, atol=0)
                fmax = 448.0 if dtype == torch.float8_e4m3fn else 57344.0
                qr = (x.float() / scale.reshape(())).clamp(-fmax, fmax).to(dtype)
            d = (q.float() - qr.float()).abs()
            # identical except where bf16 -> scaled value lands exactly between two codes (none expected), so exact
            assert float(d.max()) == 0.0, (float(d.max()), int((d > 0).sum()))
    _no_kernel_errors()


def test_fp8_linear_uses_native_quantisation(ops):
    """Float8 rowwise linear: forward, input gradient and weight gradient all reach the 8-bit tcgen05 GEMM with natively
    quantised operands and agree with the bf16 layer within float8 error."""
    from torchtitan_b200.ops.quant import QuantRecipe, quant_linear

    torch.manual_seed(0)
    x = torch.randn(2, 256, 512, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(384, 512, device="cuda") * 0.05).bfloat16().requires_grad_()
    for scaling in ("rowwise", "tensorwise"):
        x.grad = w.grad = None
        y = quant_linear(x, w, None, QuantRecipe(kind="float8", scaling=scaling))
        g = torch.randn_like(y)
        y.backward(g)
        xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
        yr = xr @ wr.t()
        yr.backward(g.float())
        assert _rel(y, yr) < 6e-2, _rel(y, yr)
        assert _rel(x.grad, xr.grad) < 8e-2, _rel(x.grad, xr.grad)
        assert _rel(w.grad, wr.grad) < 8e-2, _rel(w.grad, wr.grad)
    _no_kernel_errors()


def test_mxfp8_quantise_kernels(ops):
    """Native MXFP8 quantisation (e4m3 data, one E8M0 exponent per 32 elements of the contraction, RCEIL) of an operand
    as stored and as a transposed view: exponents and codes equal the elementwise definition."""
    from torchtitan_b200.ops import cuda_ops
    from torchtitan_b200.ops.quant import dequantize_mxfp8, quantize_mxfp8

    torch.manual_seed(0)
    for R, K in [(256, 1024), (136, 96)]:
        base = (torch.randn(R, K, device="cuda") * torch.exp(torch.randn(R, 1, device="cuda") * 4)).bfloat16()
        base[5, :64] = 0                                               # all-zero blocks take the exponent floor
        for x in (base, (torch.randn(K, R, device="cuda") * 5).bfloat16().t()):
            got = cuda_ops.quantize_mxfp8_operand(x)
            assert got is not None
            q, sc = got
            qr, sr = quantize_mxfp8(x.contiguous())
            assert torch.equal(sc, sr), (sc.flatten()[:8], sr.flatten()[:8])
            assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
            back = dequantize_mxfp8(q, sc)
            assert _rel(back, x.float()) < 7e-2       # e4m3 keeps 3 mantissa bits: up to 2^-4 of the block maximum
    _no_kernel_errors()


@pytest.mark.parametrize("pair", [1, 0])
@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 512), (384, 768, 1024), (200, 328, 224), (4096, 4096, 2048),
                                   (520, 1000, 384)])
def test_gemm_mxfp8_block_scaled(ops, M, N, K, pair):
    """Block-scaled tcgen05 MXFP8 GEMM (scales applied by the MMA) vs the fp32 product of the dequantised operands, with
    CTA-pair tiles (the default for shapes of at least 256 x 256) and with the single-CTA kernel."""
    from torchtitan_b200.ops import native, quant

    if not native.has("tt_gemm_mxfp8"):
        pytest.skip("library built without tt_gemm_mxfp8")
    if native.has("tt_gemm_mx_set_pair"):
        native.lib().tt_gemm_mx_set_pair(pair)
    elif pair == 0:
        pytest.skip("library has one MXFP8 kernel only")
    torch.manual_seed(0)
    # rows and K blocks of very different magnitude, so that a misplaced scale shows
    a = torch.randn(M, K, device="cuda") * torch.exp2(torch.randint(-6, 7, (M, K // 32), device="cuda").float()).repeat_interleave(32, 1)
    b = torch.randn(N, K, device="cuda") * torch.exp2(torch.randint(-6, 7, (N, K // 32), device="cuda").float()).repeat_interleave(32, 1)
    qa, sa = quant.quantize_mxfp8(a.bfloat16())
    qb, sb = quant.quantize_mxfp8(b.bfloat16())
    want = quant.dequantize_mxfp8(qa, sa) @ quant.dequantize_mxfp8(qb, sb).t()
    got = ops.gemm_mxfp8(qa, qb, sa, sb, torch.float32)
    _no_kernel_errors()
    assert _rel(got, want) < 1e-3, _rel(got, want)
    got16 = ops.gemm_mxfp8(qa, qb, sa, sb, torch.bfloat16)
    if native.has("tt_gemm_mx_set_pair"):
        native.lib().tt_gemm_mx_set_pair(1)
    assert _rel(got16, want) < 1e-2


@pytest.mark.parametrize("rows,K,N", [(256, 256, 512), (512, 1024, 768), (96, 160, 224)])
def test_mx_linear_op_matches_definition(ops, rows, K, N):
    """The MXFP8 linear as one op (quantise with scales in the MMA's layout + block-scaled GEMM, weight gradient into a
    gradient slot) against the PyTorch definition of the same arithmetic (quantise, dequantise, fp32 matmul), forward,
    input gradient and weight gradient; operands with block-dependent magnitudes so that a misplaced scale shows."""
    from torchtitan_b200.ops import native, quant

    if not native.has("tt_mxfp8_quant_rows_swz"):
        pytest.skip("library built without the swizzled MXFP8 quantisers")
    torch.manual_seed(0)
    mag = lambda r, c: torch.exp2(torch.randint(-4, 5, (r, c // 32), device="cuda").float()).repeat_interleave(32, 1)
    x = (torch.randn(rows, K, device="cuda") * mag(rows, K)).bfloat16().requires_grad_()
    w = (torch.randn(N, K, device="cuda") * 0.05 * mag(N, K)).bfloat16().requires_grad_()
    y = ops.mx_linear(x.view(1, rows, K), w)
    assert y is not None and y.shape == (1, rows, N)
    gy = (torch.randn(1, rows, N, device="cuda") * mag(rows, N).view(1, rows, N)).bfloat16()
    y.backward(gy)
    _no_kernel_errors()

    def mm(a, b_t):           # the definition: both operands block-scaled along the contraction
        qa, sa = quant.quantize_mxfp8(a.contiguous())
        qb, sb = quant.quantize_mxfp8(b_t.contiguous())
        return quant.dequantize_mxfp8(qa, sa) @ quant.dequantize_mxfp8(qb, sb).t()

    xd, wd, g2 = x.detach(), w.detach(), gy.view(rows, N)
    assert _rel(y.view(rows, N), mm(xd, wd)) < 1e-2
    assert _rel(x.grad, mm(g2, wd.t())) < 1e-2
    assert _rel(w.grad, mm(g2.t(), xd.t())) < 1e-2
    # and close to the unquantised product (e4m3 keeps 3 mantissa bits)
    assert _rel(y.view(rows, N), xd.float() @ wd.float().t()) < 8e-2

@pytest.mark.parametrize("weighted", [True, False])
def test_moe_gather_and_combine_kernels_match_indexing(ops, weighted):
    """Routed-token gather (``x[order // k]``) and the un-sort + sum over a token's k copies through the fused row kernels,
    against plain indexing in fp32, with gradients; and the masked copy used to leave a communication buffer."""
    torch.manual_seed(0)
    T, k, D = 300, 4, 256
    order = torch.randperm(T * k, device="cuda")
    x = torch.randn(T, D, device="cuda").bfloat16().requires_grad_()
    w = torch.rand(T, k, device="cuda").requires_grad_() if weighted else None
    rows = ops.moe_gather_rows(x, order, k)
    out = ops.moe_scatter_combine(rows * 1.0, order, w, T, k)
    g = torch.randn_like(out)
    out.backward(g)
    _no_kernel_errors()
    xf = x.detach().float().requires_grad_()
    wf = w.detach().clone().requires_grad_() if weighted else None
    rf = xf[order // k]
    uns = torch.zeros(T * k, D, device="cuda").index_copy(0, order, rf).view(T, k, D)
    ref = (uns * wf.unsqueeze(-1)).sum(1) if weighted else uns.sum(1)
    ref.backward(g.float())
    assert torch.equal(rows.detach(), x.detach()[order // k])
    assert _rel(out, ref) < 1e-2 and _rel(x.grad, xf.grad) < 2e-2
    if weighted:
        assert _rel(w.grad, wf.grad) < 2e-2
    keep = torch.rand(T * k, device="cuda") > 0.3
    got = ops.copy_rows_where(rows.detach(), keep)
    assert torch.equal(got, torch.where(keep.unsqueeze(1), rows.detach(), torch.zeros((), dtype=torch.bfloat16, device="cuda")))



def test_scale_rows_fused(ops):
    """Rows times one fp32 factor each in one pass, with both gradients, against the fp32 definition."""
    torch.manual_seed(0)
    rows = torch.randn(1000, 2048, device="cuda").bfloat16().requires_grad_()
    sc = torch.rand(1000, 1, device="cuda").requires_grad_()
    out = ops.scale_rows(rows, sc)
    g = torch.randn_like(out)
    out.backward(g)
    _no_kernel_errors()
    rf, sf = rows.detach().float().requires_grad_(), sc.detach().clone().requires_grad_()
    ref = rf * sf
    ref.backward(g.float())
    assert _rel(out, ref) < 1e-2 and _rel(rows.grad, rf.grad) < 1e-2
    assert _rel(sc.grad, sf.grad) < 1e-2 and sc.grad.shape == sc.shape


@pytest.mark.parametrize("sizes,K,N", [
    ([128, 0, 384, 256], 256, 384),          # an empty expert, N % 256 == 128 (the last tile hangs over the next expert)
    ([256, 128, 128, 0, 0, 512, 128, 128], 768, 2048),   # Qwen3-30B-A3B down projection
    ([640], 2048, 768),
])
def test_mx_grouped_linear_matches_definition(ops, sizes, K, N):
    """Routed-expert linear in MXFP8 as three grouped launches (forward, input gradient, weight gradient) with the group
    boundaries on the device, against the PyTorch definition expert by expert (quantise along each GEMM's contraction,
    dequantise, fp32 matmul). Buffer rows past the last group stay zero."""
    from torchtitan_b200.ops import native, quant

    if not native.has("tt_grouped_gemm_mxfp8"):
        pytest.skip("library built without the grouped MXFP8 GEMM")
    torch.manual_seed(0)
    G, used = len(sizes), sum(sizes)
    R = used + 128                                            # the dispatcher's buffer is longer than the rows in use
    mag = lambda r, c: torch.exp2(torch.randint(-3, 4, (r, c // 32), device="cuda").float()).repeat_interleave(32, 1)
    x = torch.zeros(R, K, device="cuda")
    x[:used] = torch.randn(used, K, device="cuda") * mag(used, K)
    x = x.bfloat16().requires_grad_()
    w = (torch.randn(G, N, K, device="cuda") * 0.05 * mag(G * N, K).view(G, N, K)).bfloat16().requires_grad_()
    counts = torch.tensor(sizes, device="cuda", dtype=torch.int64)
    counts._tt_aligned = 128
    y = ops.mx_grouped_linear(x, w, counts)
    assert y is not None and y.shape == (R, N)
    gy = torch.zeros(R, N, device="cuda")
    gy[:used] = torch.randn(used, N, device="cuda") * mag(used, N)
    gy = gy.bfloat16()
    y.backward(gy)
    _no_kernel_errors()

    def mm(a, b_t):
        qa, sa = quant.quantize_mxfp8(a.contiguous())
        qb, sb = quant.quantize_mxfp8(b_t.contiguous())
        return quant.dequantize_mxfp8(qa, sa) @ quant.dequantize_mxfp8(qb, sb).t()

    xd, wd = x.detach(), w.detach()
    y_ref, gx_ref, gw_ref = torch.zeros(R, N, device="cuda"), torch.zeros(R, K, device="cuda"), torch.zeros(G, N, K, device="cuda")
    s = 0
    for g, n in enumerate(sizes):
        if n:
            y_ref[s:s + n] = mm(xd[s:s + n], wd[g])
            gx_ref[s:s + n] = mm(gy[s:s + n], wd[g].t())
            gw_ref[g] = mm(gy[s:s + n].t(), xd[s:s + n].t())
        s += n
    assert _rel(y, y_ref) < 1e-2
    assert _rel(x.grad, gx_ref) < 1e-2
    assert _rel(w.grad, gw_ref) < 1e-2
    assert float(y[used:].abs().max()) == 0.0 and float(x.grad[used:].abs().max()) == 0.0
    for g, n in enumerate(sizes):
        if n == 0:
            assert float(w.grad[g].abs().max()) == 0.0

@pytest.mark.parametrize("M,N,K", [(256, 512, 192), (200, 264, 136), (4096, 4096, 1024), (96, 128, 64)])
def test_gemm_with_residual_in_the_epilogue(ops, M, N, K):
    """``x W^T + r`` in one kernel (the block's skip connection added by the output projection) against the fp32
    definition, forward and all three gradients; both the CTA-pair and the single-CTA kernel sizes."""
    torch.manual_seed(0)
    x = torch.randn(2, M // 2, K, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16().requires_grad_()
    r = torch.randn(2, M // 2, N, device="cuda").bfloat16().requires_grad_()
    y = ops.linear_residual(x, w, r)
    assert y is not None and y.shape == r.shape
    gy = torch.randn_like(y)
    y.backward(gy)
    _no_kernel_errors()
    want = x.detach().float() @ w.detach().float().t() + r.detach().float()
    assert _rel(y, want) < 1e-2
    # the addition happens in fp32 before the single rounding to bf16
    assert (y.float() - want).abs().max() <= want.abs().max() * 2 ** -8 + 1e-6
    assert torch.equal(r.grad, gy)
    assert _rel(x.grad, gy.float() @ w.detach().float()) < 1e-2
    assert _rel(w.grad, gy.flatten(0, 1).float().t() @ x.detach().flatten(0, 1).float()) < 1e-2


def test_linears_of_one_input_share_their_input_gradient(ops):
    """``wq / wk / wv`` as one autograd node: outputs as separate linears, the input gradient summed inside the GEMMs."""
    torch.manual_seed(0)
    x = torch.randn(2, 192, 512, device="cuda").bfloat16().requires_grad_()
    ws = [(torch.randn(n, 512, device="cuda") * 0.05).bfloat16().requires_grad_() for n in (512, 128, 128)]
    ys = ops.multi_linear(x, ws)
    assert ys is not None and [y.shape[-1] for y in ys] == [512, 128, 128]
    gys = [torch.randn_like(y) for y in ys]
    torch.autograd.backward(ys, gys)
    _no_kernel_errors()
    xf = x.detach().float()
    want_gx = sum(g.float() @ w.detach().float() for g, w in zip(gys, ws))
    assert _rel(x.grad, want_gx) < 1.5e-2
    for y, g, w in zip(ys, gys, ws):
        assert _rel(y, xf @ w.detach().float().t()) < 1e-2
        assert _rel(w.grad, g.flatten(0, 1).float().t() @ xf.flatten(0, 1)) < 1e-2
    # one output unused: its weight gets no gradient, the others are unchanged
    x2 = x.detach().clone().requires_grad_()
    ya, yb, _ = ops.multi_linear(x2, [w.detach().requires_grad_() for w in ws])
    torch.autograd.backward([ya, yb], gys[:2])
    assert _rel(x2.grad, gys[0].float() @ ws[0].detach().float() + gys[1].float() @ ws[1].detach().float()) < 1.5e-2


def test_block_with_residual_epilogue_matches_separate_additions(ops, monkeypatch):
    """A Llama block with the skip connections folded into ``wo`` / ``w2`` and the input gradients of ``wq / wk / wv`` and
    ``w1 / w3`` summed in GEMM epilogues, against the same block with separate additions: outputs and every gradient
    agree to bf16 rounding."""
    import dataclasses

    from torchtitan_b200.models.common import linear as linear_mod
    from torchtitan_b200.models.llama3 import llama3_configs

    cfg = llama3_configs["debugmodel"]
    attn = dataclasses.replace(cfg.layer.attention, n_heads=8, n_kv_heads=2)              # head dimension 128
    cfg = dataclasses.replace(cfg, n_layers=1, dim=1024, layer=dataclasses.replace(cfg.layer, attention=attn),
                              rope=dataclasses.replace(cfg.rope, dim=128, max_seq_len=256))
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = cfg.build()
    model.init_weights()
    model = model.bfloat16()
    block = next(iter(model.layers.values()))
    x = torch.randn(2, 256, cfg.dim, device="cuda").bfloat16()
    gy = torch.randn_like(x)
    results = []
    for on in (True, False):
        monkeypatch.setattr(linear_mod, "RESIDUAL_EPILOGUE", on)
        monkeypatch.setattr(linear_mod, "FUSED_DGRAD", on)
        block.zero_grad()
        xi = x.clone().requires_grad_()
        y = block(xi, model.freqs_cis, None)
        y.backward(gy)
        results.append((y.detach(), xi.grad, {n: p.grad.clone() for n, p in block.named_parameters()}))
    _no_kernel_errors()
    (ya, ga, pa), (yb, gb, pb) = results
    assert _rel(ya, yb) < 1e-2 and _rel(ga, gb) < 1e-2
    for n in pa:
        assert _rel(pa[n], pb[n]) < 2e-2, n


@pytest.mark.parametrize("Dqk,Dv,H,Hkv", [(64, 64, 8, 2), (192, 128, 4, 4), (128, 128, 4, 2)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_forward_head_dims(ops, Dqk, Dv, H, Hkv, causal):
    """Forward kernel instantiations for GPT-OSS (64/64) and multi-head latent attention (192 query/key, 128 value)."""
    from torchtitan_b200.ops import native

    if not native.has("tt_attn_fwd_dims"):
        pytest.skip("library built without tt_attn_fwd_dims")
    torch.manual_seed(0)
    B, S = 2, 512
    q = torch.randn(B, S, H, Dqk, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, Dqk, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, Dv, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(Dqk)
    o, lse = torch.ops.tt_b200.attention_fwd(q, k, v, causal, scale)
    _no_kernel_errors()
    g = H // Hkv
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float().repeat_interleave(g, 2)) * scale
    if causal:
        s = s.masked_fill(torch.ones(S, S, device="cuda", dtype=torch.bool).triu(1), float("-inf"))
    want = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float().repeat_interleave(g, 2))
    assert o.shape == (B, S, H, Dv)
    assert _rel(o, want) < 2e-2, _rel(o, want)
    assert (lse - torch.logsumexp(s, -1)).abs().max() < 2e-2


@pytest.mark.parametrize("Dqk,Dv,H,Hkv", [(64, 64, 8, 2), (192, 128, 4, 4), (192, 128, 8, 2)])
@pytest.mark.parametrize("mask", ["causal", "full", "window"])
def test_attention_other_head_dims_forward_and_backward(ops, Dqk, Dv, H, Hkv, mask):
    """GPT-OSS (64/64, sliding window and sinks elsewhere) and latent-attention (192/128) head dimensions through the
    kernels, forward and backward, against the fp32 definition."""
    from torchtitan_b200.ops import native, reference as ref

    if not native.has("tt_attn_bwd_dims"):
        pytest.skip("library built without tt_attn_bwd_dims")
    torch.manual_seed(3)
    B, S = 2, 512
    q = torch.randn(B, S, H, Dqk, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, S, Hkv, Dqk, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, S, Hkv, Dv, device="cuda").bfloat16().requires_grad_()
    assert ops.attention_supported(q, k, v)
    kw = dict(causal=mask != "full", window=100 if mask == "window" else None)
    o = ops.attention(q, k, v, **kw)
    do = torch.randn_like(o)
    o.backward(do)
    _no_kernel_errors()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    # fp32 definition (masked path of the reference module; scale = 1/sqrt(Dqk))
    g = H // Hkv
    s = torch.einsum("bqhd,bkhd->bhqk", qr, kr.repeat_interleave(g, 2)) / math.sqrt(Dqk)
    idx = torch.arange(S, device="cuda")
    dead = torch.zeros(S, S, dtype=torch.bool, device="cuda")
    if kw["causal"]:
        dead |= idx.view(1, S) > idx.view(S, 1)
    if kw["window"]:
        dead |= idx.view(1, S) <= idx.view(S, 1) - kw["window"]
    orf = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s.masked_fill(dead, float("-inf")), -1), vr.repeat_interleave(g, 2))
    orf.backward(do.float())
    assert _rel(o, orf) < 2e-2, _rel(o, orf)
    assert _rel(q.grad, qr.grad) < 3e-2, _rel(q.grad, qr.grad)
    assert _rel(k.grad, kr.grad) < 3e-2, _rel(k.grad, kr.grad)
    assert _rel(v.grad, vr.grad) < 3e-2, _rel(v.grad, vr.grad)
