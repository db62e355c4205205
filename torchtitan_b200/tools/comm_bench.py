"""Micro-benchmarks of the fused compute + collective kernels, one process per GPU:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m torchtitan_b200.tools.comm_bench ag_gemm \\
        --seq 8192 --kdim 4096 --ndim 7168

``ep``: expert-parallel dispatch + combine round trip, peer-memory kernels (``csrc/ep.cu``) vs all-to-all collectives.
``gemm_rs``: row-parallel GEMM with the sequence reduce-scatter in its epilogue (``tt_gemm_reduce_scatter``) against the
GEMM followed by NCCL reduce-scatter (``--kdim`` is the full contraction, split over the ranks).
``ag_gemm``: sequence all-gather fused into the consuming GEMM (``tt_gemm_allgather_a``) against NCCL all-gather followed
by the same GEMM kernel, and against the GEMM alone on already gathered data (the lower bound). Times are CUDA events on
the launching stream, maximum over ranks; an L2-sized buffer is overwritten between timed launches. The roofline target is
the slower of FLOPs / measured bf16 peak and remote bytes / 770 GB/s (measured peer-copy bandwidth per direction).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p.get("bf16_tflops", 1590.0)), "measured"
    except Exception:
        return 1590.0, "fallback"


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    tot = 0.0
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    t = torch.tensor([tot / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def bench_ag_gemm(args):
    from torchtitan_b200.ops import cuda_ops, native
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.async_tp import AsyncTP

    world, rank = dist.get_world_size(), dist.get_rank()
    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=world, pp=1, ep=1, etp=1, world_size=world)
    atp = AsyncTP.maybe_create(pd.get_mesh("tp"))
    assert atp is not None, "peer access / native library missing"
    atp.COPY_CTAS = args.copy_ctas
    S, K, N = args.seq, args.k, args.n
    x = torch.randn(1, S // world, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    full = torch.empty(S, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(S, N, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def fused():
        atp._forward(x, w)

    def nccl_then_gemm():
        dist.all_gather_into_tensor(full, x.view(S // world, K))
        cuda_ops.gemm_into(full, w, out)

    def gemm_only():
        cuda_ops.gemm_into(full, w, out)

    t_fused = _time(fused, args.iters, flush)
    t_nccl = _time(nccl_then_gemm, args.iters, flush)
    t_gemm = _time(gemm_only, args.iters, flush)
    peak, src = _peaks()
    flops = 2.0 * S * N * K
    remote_bytes = (world - 1) / world * S * K * 2
    t_roof = max(flops / (peak * 1e12), remote_bytes / 770e9) * 1e3
    if rank == 0:
        print(json.dumps({
            "case": "ag_gemm", "world": world, "S": S, "K": K, "N": N, "copy_ctas": args.copy_ctas,
            "fused_ms": t_fused, "nccl_allgather_plus_gemm_ms": t_nccl, "gemm_only_ms": t_gemm,
            "speedup_vs_nccl": t_nccl / t_fused, "roofline_ms": t_roof, "fraction_of_roofline": t_roof / t_fused,
            "roofline_terms": {"compute_ms": flops / (peak * 1e12) * 1e3, "nvlink_ms": remote_bytes / 770e9 * 1e3,
                               "peak_tflops": peak, "peak_source": f"of {src}"},
            "kernel_errors": native.kernel_errors(),
        }))


def bench_gemm_rs(args):
    """Row-parallel GEMM (K sharded) closed by a sequence reduce-scatter: one fused launch vs GEMM + NCCL."""
    from torchtitan_b200.ops import cuda_ops, native
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.async_tp import AsyncTP

    world, rank = dist.get_world_size(), dist.get_rank()
    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=world, pp=1, ep=1, etp=1, world_size=world)
    atp = AsyncTP.maybe_create(pd.get_mesh("tp"))
    assert atp is not None, "peer access / native library missing"
    S, K, N = args.seq, args.k // world, args.n          # K is the full contraction; each rank holds K / world
    h = torch.randn(1, S, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    part = torch.empty(S, N, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(S // world, N, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def fused():
        atp._forward_rs(h, w)

    def gemm_then_nccl():
        cuda_ops.gemm_into(h.view(S, K), w, part)
        dist.reduce_scatter_tensor(out, part)

    def gemm_only():
        cuda_ops.gemm_into(h.view(S, K), w, part)

    t_fused = _time(fused, args.iters, flush)
    t_nccl = _time(gemm_then_nccl, args.iters, flush)
    t_gemm = _time(gemm_only, args.iters, flush)
    peak, src = _peaks()
    flops = 2.0 * S * N * K
    remote_bytes = (world - 1) / world * S * N * 2
    t_roof = max(flops / (peak * 1e12), remote_bytes / 770e9) * 1e3
    if rank == 0:
        print(json.dumps({
            "case": "gemm_rs", "world": world, "S": S, "K_per_rank": K, "N": N,
            "fused_ms": t_fused, "gemm_plus_nccl_reduce_scatter_ms": t_nccl, "gemm_only_ms": t_gemm,
            "speedup_vs_nccl": t_nccl / t_fused, "roofline_ms": t_roof, "fraction_of_roofline": t_roof / t_fused,
            "roofline_terms": {"compute_ms": flops / (peak * 1e12) * 1e3, "nvlink_ms": remote_bytes / 770e9 * 1e3,
                               "peak_tflops": peak, "peak_source": f"of {src}"},
            "kernel_errors": native.kernel_errors(),
        }))


def bench_ep(args):
    """Expert-parallel dispatch + combine round trip (forward): the peer-memory kernels vs all-to-all collectives with their
    device-to-host read of the split sizes. Tokens per rank = --seq, width = --kdim, experts = --experts, top-k = --topk."""
    from torchtitan_b200.ops import native
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.parallel.ep import AllToAllDispatcher
    from torchtitan_b200.parallel.nvlink_ep import NvlinkDispatcher

    world, rank = dist.get_world_size(), dist.get_rank()
    pd = ParallelDims(dp_replicate=1, dp_shard=world, cp=1, tp=1, pp=1, ep=world, etp=1, world_size=world)
    mesh = pd.get_mesh("ep")
    assert NvlinkDispatcher.available(mesh), "peer access / native library missing"
    T, D, E, k = args.seq, args.k, args.experts, args.topk
    g = torch.Generator(device="cuda").manual_seed(rank)
    x = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    idx = torch.stack([torch.randperm(E, device="cuda", generator=g)[:k] for _ in range(64)]).repeat(T // 64 + 1, 1)[:T]
    order = torch.argsort(idx.flatten(), stable=True)
    counts = torch.bincount(idx.flatten(), minlength=E)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    res = {}
    for name, disp in (("nvlink", NvlinkDispatcher(mesh, E, alignment=64)), ("all_to_all", AllToAllDispatcher(mesh, E, alignment=64))):
        def round_trip():
            with torch.no_grad():
                rows, sizes, ctx = disp.dispatch(x, order, counts, k)
                return disp.combine(rows, ctx)
        back = round_trip()
        assert torch.equal(back, x[order // k]), name            # every row comes home unchanged
        res[name + "_ms"] = _time(round_trip, args.iters, flush)
    n = T * k
    remote = (world - 1) / world * n * D * 2 * 2                  # bytes this rank sends (dispatch) + gets back (combine)
    if rank == 0:
        print(json.dumps({
            "case": "ep_dispatch_combine", "world": world, "tokens_per_rank": T, "top_k": k, "experts": E, "width": D,
            **res, "speedup_vs_all_to_all": res["all_to_all_ms"] / res["nvlink_ms"],
            "nvlink_roofline_ms": remote / 2 / 770e9 * 1e3 * 2, "rows": n, "kernel_errors": native.kernel_errors(),
        }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["ag_gemm", "gemm_rs", "ep"])
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--kdim", dest="k", type=int, default=4096)
    ap.add_argument("--ndim", dest="n", type=int, default=7168)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--copy-ctas", type=int, default=16)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    args = ap.parse_args()
    rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    try:
        {"ag_gemm": bench_ag_gemm, "gemm_rs": bench_gemm_rs, "ep": bench_ep}[args.what](args)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
