"""Peer-memory collective kernels, checked on one GPU by giving the kernel W local buffers as
"peers" (flags already at the expected version, so nothing waits on another launch)."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr_array(tensors):
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p)), arr


@pytest.fixture(scope="module")
def L():
    from torchtitan_b200.ops import native
    from torchtitan_b200.parallel import nvlink_comm  # registers the comm symbols

    return native.lib()


@pytest.mark.parametrize("W", [2, 4, 8])
def test_allgather_and_reduce_scatter_kernels(L, W):
    torch.manual_seed(0)
    dev = "cuda"
    stream = torch.cuda.current_stream().cuda_stream
    # three "parameters": rows x inner, chunked over W ranks (one with an odd tail)
    shapes = [(64 * W, 256), (8 * W, 40), (W, 7)]
    segs, s_off, f_off = [], 0, 0
    for rows, inner in shapes:
        chunk = rows // W * inner
        segs.append((s_off, f_off, chunk))
        s_off += (chunk + 7) // 8 * 8
        f_off += (W * chunk + 7) // 8 * 8
    seg_t = torch.tensor(segs, dtype=torch.int64, device=dev)
    shards = [torch.randn(s_off, device=dev).bfloat16() for _ in range(W)]
    flags = [torch.full((1,), 3, dtype=torch.int32, device=dev) for _ in range(W)]
    for my_rank in (0, W - 1):
        dst = torch.zeros(f_off, device=dev, dtype=torch.bfloat16)
        p, k1 = _ptr_array(shards)
        f, k2 = _ptr_array(flags)
        assert L.tt_allgather_pull(p, f, seg_t.data_ptr(), len(segs), dst.data_ptr(), W, my_rank, 3, 0, 4, stream) == 0
        torch.cuda.synchronize()
        for (so, fo, chunk) in segs:
            want = torch.cat([sh[so : so + chunk] for sh in shards])
            assert torch.equal(dst[fo : fo + W * chunk], want)
    # reduce-scatter: every "peer" has a full staging buffer
    staging = [torch.randn(f_off, device=dev).bfloat16() for _ in range(W)]
    for my_rank in (0, W - 1):
        out = torch.full((s_off,), 5.0, device=dev)
        p, k1 = _ptr_array(staging)
        f, k2 = _ptr_array(flags)
        assert L.tt_reduce_scatter_pull(p, f, seg_t.data_ptr(), len(segs), out.data_ptr(), W, my_rank, 3, 0, 8, stream) == 0
        assert L.tt_reduce_scatter_pull(p, f, seg_t.data_ptr(), len(segs), out.data_ptr(), W, my_rank, 3, 1, 8, stream) == 0
        torch.cuda.synchronize()
        for (so, fo, chunk) in segs:
            want = sum(st[fo + my_rank * chunk : fo + (my_rank + 1) * chunk].float() for st in staging)
            assert torch.allclose(out[so : so + chunk], 2 * want, rtol=1e-6, atol=1e-6)
    err = (ctypes.c_int * 4)()
    assert L.tt_comm_error(err) == 0


def test_bounded_wait_reports_missing_flag(L):
    """A peer flag that never reaches the expected version: the kernel gives up after the limit,
    records {code, peer, expected, seen}, leaves the output untouched and the context usable."""
    dev = "cuda"
    stream = torch.cuda.current_stream().cuda_stream
    W = 2
    assert L.tt_comm_set_wait_ns(200_000_000) == 0  # 0.2 s
    try:
        shards = [torch.ones(64, device=dev).bfloat16() for _ in range(W)]
        flags = [torch.full((1,), 7, dtype=torch.int32, device=dev), torch.full((1,), 2, dtype=torch.int32, device=dev)]
        seg_t = torch.tensor([[0, 0, 64]], dtype=torch.int64, device=dev)
        dst = torch.zeros(128, device=dev, dtype=torch.bfloat16)
        p, k1 = _ptr_array(shards)
        f, k2 = _ptr_array(flags)
        assert L.tt_allgather_pull(p, f, seg_t.data_ptr(), 1, dst.data_ptr(), W, 0, 7, 0, 2, stream) == 0
        torch.cuda.synchronize()
        err = (ctypes.c_int * 4)()
        assert L.tt_comm_error(err) == 1
        assert (err[1], err[2], err[3]) == (1, 7, 2)
        assert float(dst.float().abs().sum()) == 0.0
        assert L.tt_comm_error(err) == 0  # reading cleared it
        # the context is still healthy
        assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    finally:
        L.tt_comm_set_wait_ns(20_000_000_000)


def test_fused_allgather_gemm_single_gpu_emulation(L):
    """All-gather fused into the GEMM, with the "peers" being local buffers whose flags are already published (so no CTA
    waits on another launch): remote slices are pulled by the copy CTAs of the same launch while the GEMM CTAs multiply."""
    _fused_case(L, 4, 256, 512, 768)      # whole 256-row tiles per rank: CTA-pair kernel
    _fused_case(L, 4, 128, 320, 264)      # single-CTA tile kernel, ragged N and K
    _fused_case(L, 2, 256, 512, 768, b_mn=True)   # weight read as [contraction, output]: the backward form
    _fused_case(L, 2, 128, 192, 320, b_mn=True)


def _fused_case(L, W, rows_local, K, N, b_mn=False):
    torch.manual_seed(0)
    M = W * rows_local
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    want = x.float() @ w.float().t()
    wb = w.t().contiguous() if b_mn else w                  # [K, N] when read as [contraction, output]
    for rank in (0, W - 1):
        # rank r's buffer holds only its own slice; the others are garbage until pulled
        bufs = []
        for r in range(W):
            b = torch.full((M, K), float("nan"), device="cuda", dtype=torch.bfloat16)
            b[r * rows_local : (r + 1) * rows_local] = x[r * rows_local : (r + 1) * rows_local]
            bufs.append(b)
        flags = [torch.full((1,), 7, dtype=torch.int32, device="cuda") for _ in range(W)]
        ready = torch.zeros(M // 128, dtype=torch.int32, device="cuda")
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        p, k1 = _ptr_array(bufs)
        f, k2 = _ptr_array(flags)
        rc = L.tt_gemm_allgather_a(p, f, W, rank, 7, wb.data_ptr(), out.data_ptr(), M, N, K, int(b_mn), wb.stride(0), N, 0,
                                   ready.data_ptr(), 1, 8, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert L.tt_gemm_error() == 0
        assert torch.equal(bufs[rank], x)                       # the gathered operand is complete locally afterwards
        assert (ready == 1).all()
        err = (out.float() - want).abs().max() / want.abs().max()
        assert err < 1e-2, err


def test_fused_gemm_reduce_scatter_single_gpu_emulation(L):
    """GEMM with the reduce-scatter in its epilogue, the "ranks" being local buffers. Launches run one after another and
    none waits on a later one: all ranks but the last contribute only (their own rows are left out), the last one also
    computes and reduces its own rows; the next call (counters keep counting) rotates which rank goes last."""
    if not hasattr(L, "tt_gemm_reduce_scatter"):
        pytest.skip("library built without tt_gemm_reduce_scatter")
    for mode in (0, 1):                  # peer-owned tiles first / interleaved tile order
        L.tt_gemm_rs_set_interleave(mode)
        _rs_case(L, 2, 512, 256, 768)
        _rs_case(L, 4, 128, 192, 264)
    L.tt_gemm_rs_set_interleave(-1)
    _rs_case(L, 2, 512, 256, 768)        # whole 256-row tiles per rank: CTA-pair kernel
    _rs_case(L, 2, 256, 128, 328)        # CTA-pair kernel, ragged last column tile (72 columns)
    _rs_case(L, 4, 128, 192, 264)        # single-CTA tile kernel, ragged N tile
    _rs_case(L, 1, 256, 128, 512)        # one rank: staging round trip only
    _rs_case(L, 2, 256, 192, 512, b_mn=True)     # weight read as [contraction, output]: the backward form


def _rs_case(L, W, rows_per_rank, Kshard, N, b_mn=False):
    torch.manual_seed(1)
    M = W * rows_per_rank
    stream = torch.cuda.current_stream().cuda_stream
    A = [torch.randn(M, Kshard, device="cuda").bfloat16() for _ in range(W)]
    B = [(torch.randn(N, Kshard, device="cuda") * 0.1).bfloat16() for _ in range(W)]
    parts = [a.float() @ b.float().t() for a, b in zip(A, B)]
    Bm = [b.t().contiguous() for b in B] if b_mn else B      # [Kshard, N] when read as [contraction, output]
    want = sum(parts)
    stages = [torch.full((W, rows_per_rank, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    counts = [torch.zeros(W * (rows_per_rank // 128) * ((N + 255) // 256), dtype=torch.int32, device="cuda") for _ in range(W)]
    sp, k1 = _ptr_array(stages)
    cp, k2 = _ptr_array(counts)
    for call in range(1, W + 1):
        last = (call - 1) % W
        order = [r for r in range(W) if r != last] + [last]
        out = torch.full((rows_per_rank, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        for r in order:
            rc = L.tt_gemm_reduce_scatter(A[r].data_ptr(), Bm[r].data_ptr(), sp, cp, out.data_ptr(), W, r, M, N, Kshard,
                                          Kshard, int(b_mn), Bm[r].stride(0), call, 0 if r == last else 1, stream)
            assert rc == 0
        torch.cuda.synchronize()
        assert L.tt_gemm_error() == 0
        ref = want[last * rows_per_rank : (last + 1) * rows_per_rank]
        err = (out.float() - ref).abs().max() / ref.abs().max()
        assert err < 1e-2, (W, call, err)
