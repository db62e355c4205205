"""The library's allocation-free RMSNorm-backward entry point (``tt_rmsnorm_bwd_noalloc``).

Some embedders of the native library must not allocate device memory at the call site (fixed
memory budget, a host application's capture window, an allocator owned by another runtime). For
them the library keeps the dW partial-sum scratch in a built-in device array. This test calls the
exported C symbol directly through ctypes, twice in a row, and checks both results against the
ordinary entry point that takes a caller-allocated scratch buffer. It is collected last on purpose:
if it fails, a run that stops at the first failure has already covered everything else.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from torchtitan_b200.ops import native

    L = native.lib()
    P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    L.tt_rmsnorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, LL, I, I, P]
    L.tt_rmsnorm_bwd_noalloc.restype = I
    L.tt_rmsnorm_bwd_noalloc_max_dim.argtypes = []
    L.tt_rmsnorm_bwd_noalloc_max_dim.restype = I
    L.tt_noalloc_strerror.argtypes = [I]
    L.tt_noalloc_strerror.restype = ctypes.c_char_p
    return L


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 0), (torch.float32, 1)])
def test_noalloc_matches_regular_entry_twice(dtype, code):
    L = _lib()
    dev = "cuda"
    stream = torch.cuda.current_stream().cuda_stream
    calls_done = 0
    for trial, (rows, D) in enumerate([(777, 4096), (300, 1024)]):  # two calls in a row share the array
        torch.manual_seed(trial)
        x = torch.randn(rows, D, device=dev, dtype=dtype)
        dy = torch.randn(rows, D, device=dev, dtype=dtype)
        w = (torch.randn(D, device=dev) * 0.1 + 1).to(dtype)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        # regular entry point with caller scratch
        nblk = L.tt_rmsnorm_bwd_blocks(rows, D)
        scratch = torch.empty(nblk, D, device=dev, dtype=torch.float32)
        dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
        assert L.tt_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx_ref.data_ptr(),
                                dw_ref.data_ptr(), scratch.data_ptr(), rows, D, code, stream) == 0
        # allocation-free entry point: outputs are allocated here, by the caller, before the call
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0] if calls_done else None
        rc = L.tt_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                      dw.data_ptr(), rows, D, code, stream)
        assert rc == 0, L.tt_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # PyTorch's counter only sees its own allocator: from the second call on (the module and the scratch address are
        # loaded by then) the driver's free-memory figure must not move either, so a cudaMalloc inside the library shows
        if free_before is not None:
            assert torch.cuda.mem_get_info()[0] >= free_before
        calls_done += 1
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        assert torch.allclose(dx.float(), dx_ref.float(), rtol=tol, atol=tol)
        assert torch.allclose(dw.float(), dw_ref.float(), rtol=tol, atol=tol * 10)
        # and against plain PyTorch fp32 math
        xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
        (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr).backward(dy.float())
        rel = (dx.float() - xr.grad).abs().max() / xr.grad.abs().max()
        assert rel < (3e-2 if dtype == torch.bfloat16 else 1e-4)


def test_noalloc_rejects_oversize():
    L = _lib()
    big = L.tt_rmsnorm_bwd_noalloc_max_dim() + 8
    x = torch.zeros(4, big, device="cuda")
    rstd = torch.ones(4, device="cuda")
    dx = torch.empty_like(x)
    rc = L.tt_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), None, rstd.data_ptr(), dx.data_ptr(), None, 4, big, 1,
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == -20
    assert b"exceeds" in L.tt_noalloc_strerror(rc)
