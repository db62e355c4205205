"""Micro-benchmarks of the native kernels with CUDA-event timing.

    python -m torchtitan_b200.tools.kernel_bench gemm --m 8192 --n 14336 --k 4096 [--layout nn|nt|tt] [--compare]
    python -m torchtitan_b200.tools.kernel_bench attention --seq 8192 --heads 32 --kv-heads 8 [--compare]
    python -m torchtitan_b200.tools.kernel_bench elementwise

Each case is warmed up, then timed over ``--iters`` launches on the current stream; between timed
launches a buffer larger than L2 is overwritten so every launch starts cold. ``--compare`` also
times the PyTorch library op (cuBLAS / SDPA) for reference. Prints one JSON line per case.
"""

from __future__ import annotations

import argparse
import json
import math

import torch


class Timer:
    def __init__(self, flush_mb: int = 256):
        self.flush = torch.empty(flush_mb * 1024 * 1024, dtype=torch.uint8, device="cuda")

    def time(self, fn, iters: int, warmup: int = 3) -> float:
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(iters):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / iters


def bench_gemm(args, timer):
    from torchtitan_b200.ops import cuda_ops

    M, N, K = args.m, args.n, args.k
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    lay = args.layout
    a_mn, b_mn = lay in ("tt",), lay in ("nt", "tt")
    A = a.t().contiguous() if a_mn else a
    B = b.t().contiguous() if b_mn else b
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = timer.time(lambda: cuda_ops.gemm_into(A, B, out, a_mn=a_mn, b_mn=b_mn), args.iters)
    res = {"case": f"gemm_{lay}", "M": M, "N": N, "K": K, "ms": ms, "tflops": 2 * M * N * K / ms / 1e9}
    if args.compare:
        if lay == "nn":
            f = lambda: torch.matmul(a, b.t(), out=out)
        elif lay == "nt":
            f = lambda: torch.matmul(a, B, out=out)
        else:
            f = lambda: torch.matmul(A.t(), B, out=out)
        ms2 = timer.time(f, args.iters)
        res.update({"cublas_ms": ms2, "cublas_tflops": 2 * M * N * K / ms2 / 1e9, "ratio_vs_cublas": ms2 / ms})
    return res


def bench_gemm_fp8(args, timer):
    """float8 (e4m3, rowwise scales) GEMM through the tcgen05 kind::f8f6f4 path; ``--compare`` adds torch._scaled_mm."""
    from torchtitan_b200.ops import cuda_ops, quant

    M, N, K = args.m, args.n, args.k
    qa, sa = quant.quantize_fp8(torch.randn(M, K, device="cuda"), -1)
    qb, sb = quant.quantize_fp8(torch.randn(N, K, device="cuda"), -1)
    ms = timer.time(lambda: cuda_ops.gemm_fp8(qa, qb, sa, sb, torch.bfloat16), args.iters)
    res = {"case": "gemm_fp8_rowwise", "M": M, "N": N, "K": K, "ms": ms, "tflops": 2 * M * N * K / ms / 1e9}
    if args.compare:
        f = lambda: torch._scaled_mm(qa, qb.t(), scale_a=sa.float().view(M, 1), scale_b=sb.float().view(1, N), out_dtype=torch.bfloat16)
        try:
            ms2 = timer.time(f, args.iters)
            res.update({"cublaslt_ms": ms2, "cublaslt_tflops": 2 * M * N * K / ms2 / 1e9, "ratio_vs_cublaslt": ms2 / ms})
        except Exception as e:  # library variant not available for this shape / scaling
            res["cublaslt_error"] = str(e)[:200]
    return res


def bench_gemm_mxfp8(args, timer):
    """MXFP8 GEMM on the block-scaled tcgen05 path (scales applied by the MMA), plus the quantise kernels that feed it
    (bf16 -> e4m3 + E8M0, as stored and transposed) and the float8 rowwise quantise kernel, in GB/s of bf16 input."""
    from torchtitan_b200.ops import cuda_ops

    M, N, K = args.m, args.n, args.k
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    from torchtitan_b200.ops import native

    qa, sa = cuda_ops.quantize_mxfp8_operand(a)
    qb, sb = cuda_ops.quantize_mxfp8_operand(b)
    # the GEMM alone: operands quantised once with their scales already in the MMA's layout
    (A8, swa), (B8, swb) = cuda_ops._mx_operand(a, False), cuda_ops._mx_operand(b, False)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    L = native.lib()
    stream = torch.cuda.current_stream().cuda_stream

    def raw():
        native.check(L.tt_gemm_mxfp8(A8.data_ptr(), B8.data_ptr(), swa.data_ptr(), swb.data_ptr(), out.data_ptr(), M, N, K,
                                     A8.stride(0), B8.stride(0), out.stride(0), 0, stream), "tt_gemm_mxfp8")

    res = {"case": "gemm_mxfp8_block_scaled", "M": M, "N": N, "K": K}
    for name, pair in (("cta_pair", 1), ("single_cta", 0)):
        if native.has("tt_gemm_mx_set_pair"):
            L.tt_gemm_mx_set_pair(pair)
        elif pair:
            continue
        ms = timer.time(raw, args.iters)
        res.update({f"{name}_ms": ms, f"{name}_tflops": 2 * M * N * K / ms / 1e9})
    if native.has("tt_gemm_mx_set_pair"):
        L.tt_gemm_mx_set_pair(1)
    ms = timer.time(lambda: cuda_ops.gemm_mxfp8(qa, qb, sa, sb, torch.bfloat16), args.iters)
    res.update({"with_scale_relayout_launches_ms": ms})
    at = torch.randn(K, M, device="cuda").bfloat16().t()
    for name, fn in (("mx_quant_rows", lambda: cuda_ops.quantize_mxfp8_operand(a)),
                     ("mx_quant_transposed", lambda: cuda_ops.quantize_mxfp8_operand(at)),
                     ("fp8_quant_rows", lambda: cuda_ops.quantize_fp8_operand(a, True)),
                     ("fp8_quant_transposed", lambda: cuda_ops.quantize_fp8_operand(at, True))):
        t = timer.time(fn, args.iters)
        res[name + "_ms"] = t
        res[name + "_gbs_in"] = M * K * 2 / t / 1e6
    return res


def bench_ag_gemm(args, timer):
    """Fused all-gather GEMM on ONE GPU: the "peers" are local buffers whose flags are already published, so the copy CTAs
    and the GEMM CTAs of the single launch do all the work (intra-GPU copies stand in for NVLink loads)."""
    import ctypes

    from torchtitan_b200.ops import native

    L = native.lib()
    W, M, N, K = args.world, args.m, args.n, args.k
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    rows = M // W
    bufs = []
    for r in range(W):
        b = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
        b[r * rows : (r + 1) * rows] = x[r * rows : (r + 1) * rows]
        bufs.append(b)
    flags = [torch.full((1,), 1 << 30, dtype=torch.int32, device="cuda") for _ in range(W)]
    ready = torch.zeros(M // 128, dtype=torch.int32, device="cuda")
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    pa = (ctypes.c_void_p * W)(*[b.data_ptr() for b in bufs])
    fa = (ctypes.c_void_p * W)(*[f.data_ptr() for f in flags])
    st = torch.cuda.current_stream().cuda_stream
    ver = [0]

    def run():
        ver[0] += 1
        native.check(L.tt_gemm_allgather_a(pa, fa, W, 0, 1, w.data_ptr(), out.data_ptr(), M, N, K, 0, K, N, 0, ready.data_ptr(),
                                           ver[0], args.copy_ctas, st), "tt_gemm_allgather_a")

    ms = timer.time(run, args.iters)
    err = ((out.float() - x.float() @ w.float().t()).abs().max() / (x.float() @ w.float().t()).abs().max()).item()
    return {"case": "ag_gemm_one_gpu", "world": W, "M": M, "N": N, "K": K, "copy_ctas": args.copy_ctas, "ms": ms,
            "tflops": 2 * M * N * K / ms / 1e9, "gathered_bytes": (W - 1) * rows * K * 2, "max_rel_err": err}


def bench_grouped_gemm(args, timer):
    """Grouped GEMM with device-side offsets (forward + both gradients) on a Qwen3-30B-A3B-like expert shape."""
    from torchtitan_b200.ops import cuda_ops

    E, N, K, R = args.experts, args.n, args.k, args.m
    g = torch.Generator(device="cuda").manual_seed(0)
    raw = torch.rand(E, device="cuda", generator=g) + 0.2
    sizes = (raw / raw.sum() * (R - 64 * E)).long() // 64 * 64 + 64
    counts = sizes.clone()
    counts._tt_aligned = 64
    rows = int(sizes.sum())
    x = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(E, N, K, device="cuda") * 0.05).bfloat16().requires_grad_()
    from torchtitan_b200.ops import native as _native

    has_pair = _native.has("tt_grouped_gemm_set_pair")
    if has_pair:
        _native.lib().tt_grouped_gemm_set_pair(1)
    y = cuda_ops.grouped_linear(x, w, counts)
    gy = torch.randn_like(y)

    def fb():
        x.grad = w.grad = None
        cuda_ops.grouped_linear(x, w, counts).backward(gy)

    ms_f = timer.time(lambda: cuda_ops.grouped_linear(x, w, counts), args.iters)
    ms_fb = timer.time(fb, args.iters)
    fl = 2.0 * rows * N * K
    out = {"case": "grouped_gemm", "experts": E, "rows": rows, "N": N, "K": K, "fwd_ms": ms_f, "fwd_tflops": fl / ms_f / 1e9,
           "fwd_bwd_ms": ms_fb, "fwd_bwd_tflops": 3 * fl / ms_fb / 1e9, "cta_pairs": bool(has_pair)}
    if has_pair:                                     # the single-CTA kernel alone, for comparison
        _native.lib().tt_grouped_gemm_set_pair(0)
        s_f = timer.time(lambda: cuda_ops.grouped_linear(x, w, counts), args.iters)
        s_fb = timer.time(fb, args.iters)
        out.update(single_cta_fwd_ms=s_f, single_cta_fwd_tflops=fl / s_f / 1e9, single_cta_fwd_bwd_ms=s_fb,
                   single_cta_fwd_bwd_tflops=3 * fl / s_fb / 1e9)
    # the same layer in MXFP8 (groups padded to 128 rows; times include quantising both operands of every GEMM)
    sizes128 = (raw / raw.sum() * (R - 128 * E)).long() // 128 * 128 + 128
    c128 = sizes128.clone()
    c128._tt_aligned = 128
    rows128 = int(sizes128.sum())
    x8 = (torch.randn(rows128, K, device="cuda") * 0.5).bfloat16().requires_grad_()
    if cuda_ops.mx_grouped_linear(x8, w, c128) is not None:
        gy8 = torch.randn(rows128, N, device="cuda").bfloat16()
        ms8_f = timer.time(lambda: cuda_ops.mx_grouped_linear(x8, w, c128), args.iters)

        def fb8():
            x8.grad = w.grad = None
            cuda_ops.mx_grouped_linear(x8, w, c128).backward(gy8)

        ms8_fb = timer.time(fb8, args.iters)
        fl8 = 2.0 * rows128 * N * K
        out.update(mxfp8_rows=rows128, mxfp8_fwd_ms=ms8_f, mxfp8_fwd_tflops=fl8 / ms8_f / 1e9, mxfp8_fwd_bwd_ms=ms8_fb,
                   mxfp8_fwd_bwd_tflops=3 * fl8 / ms8_fb / 1e9)
    return out


def bench_paged_decode(args, timer):
    """Paged-KV decode attention: ``batch`` sequences of ``seq`` cached tokens; reports achieved KV read bandwidth."""
    from torchtitan_b200.ops import cuda_ops

    B, H, Hkv, D, bs, ctx = args.batch, args.heads, args.kv_heads, 128, 16, args.seq
    nblk = B * ((ctx + bs - 1) // bs)
    kc = torch.randn(nblk, bs, Hkv, D, device="cuda").bfloat16()
    vc = torch.randn(nblk, bs, Hkv, D, device="cuda").bfloat16()
    tables = torch.randperm(nblk, device="cuda").view(B, -1).int()
    lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    q = torch.randn(B, H, D, device="cuda").bfloat16()
    ms = timer.time(lambda: cuda_ops.paged_decode(q, kc, vc, tables, lens, D**-0.5), args.iters)
    nbytes = 2.0 * B * ctx * Hkv * D * 2
    return {"case": "paged_decode", "batch": B, "ctx": ctx, "H": H, "Hkv": Hkv, "ms": ms, "kv_gb_per_s": nbytes / ms / 1e6}


def bench_attention(args, timer):
    from torchtitan_b200.ops import cuda_ops

    B, S, H, Hkv, D = args.batch, args.seq, args.heads, args.kv_heads, 128
    q = torch.randn(B, S, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    scale = 1 / math.sqrt(D)
    fwd_flops = 4 * B * H * S * S * D / 2  # causal
    o, lse = torch.ops.tt_b200.attention_fwd(q, k, v, True, scale)
    do = torch.randn_like(o)
    ms_f = timer.time(lambda: torch.ops.tt_b200.attention_fwd(q, k, v, True, scale), args.iters)
    res = {"case": "attention_causal", "B": B, "S": S, "H": H, "Hkv": Hkv, "fwd_ms": ms_f, "fwd_tflops": fwd_flops / ms_f / 1e9}
    from torchtitan_b200.ops import native

    # one fused kernel (default; dQ added by bulk reduce copies) / deterministic dK,dV + dQ kernels; with --dq-modes also
    # the fused kernel with per-element atomics and with dQ dropped (how much of its time the dQ traffic costs)
    forms = [("fused", True, 4), ("split", False, 4)]
    if args.dq_modes:
        forms += [("fused_atomics", True, 5), ("fused_no_dq(timing aid)", True, 6), ("fused_A_from_smem", True, 0)]
    for form, fused, mode in forms:
        cuda_ops.ATTN_BWD_FUSED = fused
        native.lib().tt_attn_set_dq_mode(mode)
        ms_b = timer.time(lambda: torch.ops.tt_b200.attention_bwd(q, k, v, o, do, lse, True, scale), args.iters)
        res.update({f"bwd_{form}_ms": ms_b, f"bwd_{form}_tflops_algorithmic(2.5x fwd)": 2.5 * fwd_flops / ms_b / 1e9})
    cuda_ops.ATTN_BWD_FUSED = None
    native.lib().tt_attn_set_dq_mode(4)
    if args.compare:
        qt, kt, vt = (t.detach().transpose(1, 2).requires_grad_() for t in (q, k, v))
        f = lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True)
        ms_sf = timer.time(f, args.iters)
        out = f()
        g = torch.randn_like(out)
        ms_sb = timer.time(lambda: torch.autograd.grad(out, (qt, kt, vt), g, retain_graph=True), args.iters)
        res.update({"sdpa_fwd_ms": ms_sf, "sdpa_bwd_ms": ms_sb})
    return res


def bench_elementwise(args, timer):
    from torchtitan_b200.ops import cuda_ops

    out = []
    rows, D = 8192, 4096
    x = torch.randn(rows, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    ms = timer.time(lambda: torch.ops.tt_b200.rmsnorm_fwd(x, w, 1e-5), args.iters)
    out.append({"case": "rmsnorm_fwd", "rows": rows, "D": D, "ms": ms, "GBps": 2 * x.numel() * 2 / ms / 1e6})
    g = torch.randn(rows, 14336, device="cuda").bfloat16()
    u = torch.randn_like(g)
    ms = timer.time(lambda: torch.ops.tt_b200.swiglu_fwd(g, u), args.iters)
    out.append({"case": "swiglu_fwd", "n": g.numel(), "ms": ms, "GBps": 3 * g.numel() * 2 / ms / 1e6})
    V = 128256
    logits = torch.randn(rows, V, device="cuda").bfloat16()
    labels = torch.randint(0, V, (rows,), device="cuda")
    ms = timer.time(lambda: torch.ops.tt_b200.ce_fwd(logits, labels, -100), args.iters)
    out.append({"case": "ce_fwd", "rows": rows, "V": V, "ms": ms, "GBps": logits.numel() * 2 / ms / 1e6})
    n = 1 << 28
    p = torch.randn(n, device="cuda"); gr = torch.randn(n, device="cuda"); m = torch.zeros(n, device="cuda"); vv = torch.zeros(n, device="cuda")
    sh = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = timer.time(lambda: cuda_ops.adamw_flat(p, gr, m, vv, sh, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3), args.iters)
    out.append({"case": "adamw", "n": n, "ms": ms, "GBps": n * (4 * 4 + 3 * 4 + 2) / ms / 1e6})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemm_fp8", "gemm_mxfp8", "ag_gemm", "grouped_gemm", "paged_decode", "attention", "elementwise"])
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--copy-ctas", type=int, default=8)
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="nn", choices=["nn", "nt", "tt"],
                    help="nn: x@W^T (both K-major); nt: dgrad (B stored [K,N]); tt: wgrad (both stored transposed)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--compare", action="store_true")
    ap.add_argument("--dq-modes", action="store_true", help="attention: also time the fused backward's other dQ modes")
    ap.add_argument("--single-cta", action="store_true", help="gemm: force the single-CTA tile kernel")
    args = ap.parse_args()
    timer = Timer()
    if args.single_cta:
        from torchtitan_b200.ops import native as _n

        _n.lib().tt_gemm_set_pair(0)
    if args.what == "gemm":
        res = [bench_gemm(args, timer)]
    elif args.what == "gemm_fp8":
        res = [bench_gemm_fp8(args, timer)]
    elif args.what == "gemm_mxfp8":
        res = [bench_gemm_mxfp8(args, timer)]
    elif args.what == "ag_gemm":
        res = [bench_ag_gemm(args, timer)]
    elif args.what == "grouped_gemm":
        res = [bench_grouped_gemm(args, timer)]
    elif args.what == "paged_decode":
        res = [bench_paged_decode(args, timer)]
    elif args.what == "attention":
        res = [bench_attention(args, timer)]
    else:
        res = bench_elementwise(args, timer)
    from torchtitan_b200.ops import native

    for r in res:
        r["kernel_errors"] = native.kernel_errors()
        print(json.dumps(r))


if __name__ == "__main__":
    main()
