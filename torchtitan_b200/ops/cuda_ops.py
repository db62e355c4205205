"""CUDA implementations of the hot ops: thin ``torch.library`` custom ops (namespace
``tt_b200``) around the native kernels, plus the autograd functions that combine them.

Custom ops (rather than bare ctypes calls) make the kernels visible to dispatch-level tools:
per-op selective activation checkpointing names ``tt_b200::gemm`` and
``tt_b200::attention_fwd`` in its save list, and the profiler shows them by name.
Ops that the kernels do not cover (non-bf16 GEMMs, attention with head_dim != 128 or sequence
lengths that are not multiples of 128, masks other than causal) take a PyTorch path and say
so once in the log.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

from . import native
from . import reference as ref
from torchtitan_b200.tools.logging import logger, warn_once

_lib = native.lib
_ck = native.check


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _dt(t: Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise TypeError(f"unsupported dtype {t.dtype}")


# =============================================================================== GEMM
@torch.library.custom_op("tt_b200::gemm", mutates_args=())
def gemm(a: Tensor, b: Tensor, a_mn: bool, b_mn: bool, out_fp32: bool) -> Tensor:
    """``C[M,N] = A · B^T`` with bf16 operands. ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``),
    ``b`` is ``[N,K]`` (or ``[K,N]`` when ``b_mn``); rows may be strided."""
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    c = torch.empty((M, N), dtype=torch.float32 if out_fp32 else torch.bfloat16, device=a.device)
    _ck(_lib().tt_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, int(a_mn), a.stride(0), int(b_mn),
                            b.stride(0), c.stride(0), int(out_fp32), 0, None, 0, 0, _stream()), "tt_gemm_bf16")
    return c


@gemm.register_fake
def _(a, b, a_mn, b_mn, out_fp32):
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    return a.new_empty((M, N), dtype=torch.float32 if out_fp32 else torch.bfloat16)


def gemm_into(a: Tensor, b: Tensor, out: Tensor, *, a_mn=False, b_mn=False, accumulate=False, ready_flags=None,
              ready_value=0, max_ctas=0) -> Tensor:
    """Like :func:`gemm` but writes (or accumulates) into ``out`` (bf16 or fp32, row stride free)."""
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    assert out.shape == (M, N) and out.stride(1) == 1
    _ck(_lib().tt_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, int(a_mn), a.stride(0), int(b_mn),
                            b.stride(0), out.stride(0), int(out.dtype == torch.float32), int(accumulate),
                            _p(ready_flags), ready_value, max_ctas, _stream()), "tt_gemm_bf16")
    return out


def _gemm_ok(*ts: Tensor) -> bool:
    for t in ts:
        if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1 or t.stride(0) % 8 or t.data_ptr() % 16:
            return False
    return True


def _rows2d(x: Tensor) -> Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.stride(-1) == 1 else x2.contiguous()


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = _rows2d(x)
        y = torch.ops.tt_b200.gemm(x2, w, False, False, False)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.xshape = x.shape
        ctx.grad_slot = getattr(w, "_grad_slot", None)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = _rows2d(gy)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = torch.ops.tt_b200.gemm(g2, w, False, True, False).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            slot = ctx.grad_slot
            if slot is not None:
                # write dW straight into the unit's gradient buffer; autograd only carries a placeholder
                gemm_into(g2, x2, slot.tensor, a_mn=True, b_mn=True, accumulate=slot.begin())
                gw = _placeholder(w)
            else:
                gw = torch.ops.tt_b200.gemm(g2, x2, True, True, False)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = g2.float().sum(0).to(gy.dtype)
        return gx, gw, gb


@torch.library.custom_op("tt_b200::gemm_res", mutates_args=())
def gemm_res(a: Tensor, b: Tensor, r: Tensor) -> Tensor:
    """``C[M,N] = A[M,K] · B[N,K]^T + R[M,N]`` (bf16): the residual addition runs in the GEMM's epilogue."""
    M, K = a.shape
    N = b.shape[0]
    c = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    _ck(_lib().tt_gemm_bf16_res(a.data_ptr(), b.data_ptr(), c.data_ptr(), r.data_ptr(), M, N, K, 0, a.stride(0), 0, b.stride(0),
                                c.stride(0), r.stride(0), _stream()), "tt_gemm_bf16_res")
    return c


@gemm_res.register_fake
def _(a, b, r):
    return a.new_empty((a.shape[0], b.shape[0]), dtype=torch.bfloat16)


class _LinearResFn(torch.autograd.Function):
    """``y = x W^T + r``; backward as :class:`_LinearFn`, the residual's gradient is the output's."""

    @staticmethod
    def forward(ctx, x, w, res):
        x2, r2 = _rows2d(x), _rows2d(res)
        y = torch.ops.tt_b200.gemm_res(x2, w, r2)
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        ctx.grad_slot = getattr(w, "_grad_slot", None)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = _rows2d(gy)
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = torch.ops.tt_b200.gemm(g2, w, False, True, False).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            slot = ctx.grad_slot
            if slot is not None:
                gemm_into(g2, x2, slot.tensor, a_mn=True, b_mn=True, accumulate=slot.begin())
                gw = _placeholder(w)
            else:
                gw = torch.ops.tt_b200.gemm(g2, x2, True, True, False)
        return gx, gw, (gy if ctx.needs_input_grad[2] else None)


class _MultiLinearFn(torch.autograd.Function):
    """Several bias-free linears of one input (``wq / wk / wv``, ``w1 / w3``): ``y_i = x W_i^T``. The input gradient
    ``sum_i dy_i W_i`` is formed in one buffer, each GEMM after the first adding in its epilogue, instead of one tensor
    per layer summed by autograd (two extra passes over ``dx`` per additional layer)."""

    @staticmethod
    def forward(ctx, x, *ws):
        x2 = _rows2d(x)
        ys = tuple(torch.ops.tt_b200.gemm(x2, w, False, False, False).view(*x.shape[:-1], w.shape[0]) for w in ws)
        ctx.save_for_backward(x2, *ws)
        ctx.xshape = x.shape
        ctx.slots = [getattr(w, "_grad_slot", None) for w in ws]
        return ys

    @staticmethod
    def backward(ctx, *gys):
        x2, *ws = ctx.saved_tensors
        gx = None
        gws = []
        for i, (gy, w) in enumerate(zip(gys, ws)):
            if gy is None:
                gws.append(None)
                continue
            g2 = _rows2d(gy)
            if ctx.needs_input_grad[0]:
                if gx is None:
                    gx = torch.ops.tt_b200.gemm(g2, w, False, True, False)
                else:
                    gemm_into(g2, w, gx, b_mn=True, accumulate=True)
            if ctx.needs_input_grad[1 + i]:
                slot = ctx.slots[i]
                if slot is not None:
                    gemm_into(g2, x2, slot.tensor, a_mn=True, b_mn=True, accumulate=slot.begin())
                    gws.append(_placeholder(w))
                else:
                    gws.append(torch.ops.tt_b200.gemm(g2, x2, True, True, False))
            else:
                gws.append(None)
        return (gx.view(ctx.xshape) if gx is not None else None, *gws)


def multi_linear(x: Tensor, weights: list) -> tuple | None:
    """``[x @ w^T for w in weights]`` with a shared input-gradient buffer, or None when a dtype or layout is not covered."""
    if x.dtype != torch.bfloat16 or x.shape[-1] % 8:
        return None
    for w in weights:
        if w.dtype != torch.bfloat16 or w.dim() != 2 or w.stride(1) != 1 or w.stride(0) % 8 or w.data_ptr() % 16 \
                or w.shape[0] % 8 or w.shape[1] != x.shape[-1]:
            return None
    return _MultiLinearFn.apply(x, *weights)


def linear_residual(x: Tensor, weight: Tensor, residual: Tensor) -> Tensor | None:
    """``residual + x @ weight^T`` in one kernel, or None when dtype / layout / library do not allow it."""
    if not (native.has("tt_gemm_bf16_res") and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and residual.dtype == torch.bfloat16 and weight.dim() == 2 and weight.stride(1) == 1 and weight.stride(0) % 8 == 0
            and weight.data_ptr() % 16 == 0 and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0
            and residual.shape == (*x.shape[:-1], weight.shape[0]) and residual.is_contiguous()
            and residual.data_ptr() % 16 == 0):
        return None
    return _LinearResFn.apply(x, weight, residual)


_placeholders: dict = {}


def _placeholder(w: Tensor) -> Tensor:
    """Zero-stride all-zeros tensor shaped like ``w`` (costs no memory and no launch after the first)."""
    key = (w.device, w.dtype)
    z = _placeholders.get(key)
    if z is None:
        z = _placeholders[key] = torch.zeros((), dtype=w.dtype, device=w.device)
    return z.expand(w.shape)


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2 \
            and weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0 \
            and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
        return _LinearFn.apply(x, weight, bias)
    if torch.is_autocast_enabled() and weight.dtype == torch.float32:
        return _LinearFn.apply(x.to(torch.bfloat16), weight.to(torch.bfloat16), None if bias is None else bias.to(torch.bfloat16))
    warn_once(logger, f"linear with dtypes {x.dtype}/{weight.dtype} takes the PyTorch matmul path")
    return torch.nn.functional.linear(x, weight, bias)


# =============================================================================== RMSNorm
@torch.library.custom_op("tt_b200::rmsnorm_fwd", mutates_args=())
def rmsnorm_fwd(x: Tensor, w: Tensor | None, eps: float) -> tuple[Tensor, Tensor]:
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    y = torch.empty_like(x2)
    rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    _ck(_lib().tt_rmsnorm_fwd(x2.data_ptr(), _p(w), y.data_ptr(), rstd.data_ptr(), x2.shape[0], D, eps, _dt(x), _stream()),
        "tt_rmsnorm_fwd")
    return y.view(x.shape), rstd


@rmsnorm_fwd.register_fake
def _(x, w, eps):
    return torch.empty_like(x), x.new_empty(x.numel() // x.shape[-1], dtype=torch.float32)


@torch.library.custom_op("tt_b200::rmsnorm_bwd", mutates_args=())
def rmsnorm_bwd(dy: Tensor, x: Tensor, w: Tensor | None, rstd: Tensor) -> tuple[Tensor, Tensor]:
    D = x.shape[-1]
    x2, dy2 = x.reshape(-1, D), dy.reshape(-1, D)
    rows = x2.shape[0]
    dx = torch.empty_like(x2)
    nblk = _lib().tt_rmsnorm_bwd_blocks(rows, D)
    scratch = torch.empty((nblk, D), dtype=torch.float32, device=x.device)
    dw = torch.empty(D, dtype=x.dtype, device=x.device) if w is not None else torch.empty(0, dtype=x.dtype, device=x.device)
    _ck(_lib().tt_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), _p(w), rstd.data_ptr(), dx.data_ptr(),
                              dw.data_ptr() if w is not None else None, scratch.data_ptr(), rows, D, _dt(x), _stream()),
        "tt_rmsnorm_bwd")
    return dx.view(x.shape), dw


@rmsnorm_bwd.register_fake
def _(dy, x, w, rstd):
    return torch.empty_like(x), x.new_empty(x.shape[-1] if w is not None else 0)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        xc = x if x.is_contiguous() else x.contiguous()
        y, rstd = torch.ops.tt_b200.rmsnorm_fwd(xc, w, eps)
        ctx.save_for_backward(xc, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        dx, dw = torch.ops.tt_b200.rmsnorm_bwd(dyc, x, w, rstd)
        return dx, (dw if w is not None else None), None


def rms_norm(x: Tensor, weight: Tensor | None, eps: float | None) -> Tensor:
    eps = torch.finfo(x.dtype).eps if eps is None else eps
    if x.dtype in (torch.bfloat16, torch.float32) and x.shape[-1] % 8 == 0 and (weight is None or weight.dtype == x.dtype):
        return _RMSNormFn.apply(x, weight, eps)
    if weight is not None and weight.dtype != x.dtype and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, weight.to(x.dtype), eps)
    return ref.rms_norm(x, weight, eps)


# =============================================================================== RoPE
@torch.library.custom_op("tt_b200::rope", mutates_args=())
def rope_op(x: Tensor, table: Tensor, positions: Tensor | None, layout: int, inverse: bool) -> Tensor:
    B, S, H, D = x.shape
    y = torch.empty_like(x)
    pb = 0 if positions is None else positions.shape[0]
    _ck(_lib().tt_rope(x.data_ptr(), y.data_ptr(), table.data_ptr(), _p(positions), pb, B, S, H, D, layout, int(inverse),
                       _dt(x), _stream()), "tt_rope")
    return y


@rope_op.register_fake
def _(x, table, positions, layout, inverse):
    return torch.empty_like(x)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, table, positions, layout):
        ctx.table, ctx.positions, ctx.layout = table, positions, layout
        return torch.ops.tt_b200.rope(x.contiguous(), table, positions, layout, False)

    @staticmethod
    def backward(ctx, gy):
        return torch.ops.tt_b200.rope(gy.contiguous(), ctx.table, ctx.positions, ctx.layout, True), None, None, None


def rope(x: Tensor, table: Tensor, positions: Tensor | None, layout: str) -> Tensor:
    if x.dtype not in (torch.bfloat16, torch.float32):
        return ref.rope(x, table, positions, layout)
    if table.device != x.device or table.dtype != torch.float32 or not table.is_contiguous():
        table = table.to(device=x.device, dtype=torch.float32).contiguous()
    if positions is not None:
        positions = positions.to(device=x.device, dtype=torch.int64).contiguous()
        if positions.dim() == 1:
            positions = positions.unsqueeze(0)
    return _RopeFn.apply(x, table, positions, 0 if layout == "interleaved" else 1)


# =============================================================================== SwiGLU
@torch.library.custom_op("tt_b200::swiglu_fwd", mutates_args=())
def swiglu_fwd(g: Tensor, u: Tensor) -> Tensor:
    out = torch.empty_like(g)
    _ck(_lib().tt_swiglu_fwd(g.data_ptr(), u.data_ptr(), out.data_ptr(), g.numel(), _dt(g), _stream()), "tt_swiglu_fwd")
    return out


@swiglu_fwd.register_fake
def _(g, u):
    return torch.empty_like(g)


@torch.library.custom_op("tt_b200::swiglu_bwd", mutates_args=())
def swiglu_bwd(dout: Tensor, g: Tensor, u: Tensor) -> tuple[Tensor, Tensor]:
    dg, du = torch.empty_like(g), torch.empty_like(u)
    _ck(_lib().tt_swiglu_bwd(dout.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(), _dt(g),
                             _stream()), "tt_swiglu_bwd")
    return dg, du


@swiglu_bwd.register_fake
def _(dout, g, u):
    return torch.empty_like(g), torch.empty_like(u)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        g, u = g.contiguous(), u.contiguous()
        ctx.save_for_backward(g, u)
        return torch.ops.tt_b200.swiglu_fwd(g, u)

    @staticmethod
    def backward(ctx, dout):
        g, u = ctx.saved_tensors
        return torch.ops.tt_b200.swiglu_bwd(dout.contiguous(), g, u)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    if gate.dtype in (torch.bfloat16, torch.float32) and gate.dtype == up.dtype and gate.numel() % 8 == 0:
        return _SwigluFn.apply(gate, up)
    return ref.swiglu(gate, up)


# =============================================================================== attention
@torch.library.custom_op("tt_b200::attention_fwd", mutates_args=())
def attention_fwd(q: Tensor, k: Tensor, v: Tensor, causal: bool, scale: float,
                  row_lo: Tensor | None = None, sinks: Tensor | None = None) -> tuple[Tensor, Tensor]:
    """q [B,Sq,H,Dqk], k [B,Sk,Hkv,Dqk], v [B,Sk,Hkv,Dv] -> (o [B,Sq,H,Dv], lse [B,H,Sq])."""
    B, Sq, H, D = q.shape
    Sk, Hkv, Dv = k.shape[1], k.shape[2], v.shape[3]
    o = torch.empty((B, Sq, H, Dv), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    L = _lib()
    if hasattr(L, "tt_attn_fwd_dims"):
        _ck(L.tt_attn_fwd_dims(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), _p(row_lo), _p(sinks),
                               B, Sq, Sk, H, Hkv, D, Dv, int(causal), scale, _stream()), "tt_attn_fwd_dims")
        return o, lse
    if sinks is not None:
        _ck(L.tt_attn_fwd_sinks(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), _p(row_lo),
                                sinks.data_ptr(), B, Sq, Sk, H, Hkv, D, int(causal), scale, _stream()), "tt_attn_fwd_sinks")
        return o, lse
    _ck(L.tt_attn_fwd_range(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), _p(row_lo), B, Sq, Sk,
                            H, Hkv, D, int(causal), scale, _stream()), "tt_attn_fwd")
    return o, lse


@attention_fwd.register_fake
def _(q, k, v, causal, scale, row_lo=None, sinks=None):
    return (q.new_empty((q.shape[0], q.shape[1], q.shape[2], v.shape[3])),
            q.new_empty((q.shape[0], q.shape[2], q.shape[1]), dtype=torch.float32))


# None: the fused backward kernel unless deterministic algorithms are requested; True / False force one form (tests)
ATTN_BWD_FUSED: bool | None = None


def _attn_bwd_fused() -> bool:
    if ATTN_BWD_FUSED is not None:
        return bool(ATTN_BWD_FUSED) and native.has("tt_attn_bwd_fused")
    return native.has("tt_attn_bwd_fused") and not torch.are_deterministic_algorithms_enabled()


@torch.library.custom_op("tt_b200::attention_bwd", mutates_args=())
def attention_bwd(q: Tensor, k: Tensor, v: Tensor, o: Tensor, do: Tensor, lse: Tensor, causal: bool, scale: float,
                  row_lo: Tensor | None = None, col_hi: Tensor | None = None) -> tuple[Tensor, Tensor, Tensor]:
    """Two forms: one fused kernel per key tile that also adds its share of dQ into an fp32 accumulator (default: fastest,
    dQ not bitwise reproducible), or separate dK/dV and dQ kernels without atomics (``torch.use_deterministic_algorithms``)."""
    B, Sq, H, D = q.shape
    Sk, Hkv, Dv = k.shape[1], k.shape[2], v.shape[3]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if D != 128 or Dv != 128:
        # other head dimensions: key-tile kernel for dK / dV plus query-tile kernel for dQ (no atomics, deterministic)
        scratch = torch.empty((3, B, H, Sq), dtype=torch.float32, device=q.device)
        _ck(_lib().tt_attn_bwd_dims(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                    scratch.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _p(row_lo), _p(col_hi),
                                    B, Sq, Sk, H, Hkv, D, Dv, int(causal), scale, _stream()), "tt_attn_bwd_dims")
        return dq, dk, dv
    if _attn_bwd_fused():
        scratch = torch.empty((2, B, H, Sq), dtype=torch.float32, device=q.device)
        dq_acc = torch.zeros((B, Sq, H, D), dtype=torch.float32, device=q.device)
        _ck(_lib().tt_attn_bwd_fused(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                     scratch.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                     _p(row_lo), _p(col_hi), B, Sq, Sk, H, Hkv, D, int(causal), scale, _stream()),
            "tt_attn_bwd_fused")
        return dq, dk, dv
    delta = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    _ck(_lib().tt_attn_bwd_range(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                 delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _p(row_lo), _p(col_hi), B, Sq,
                                 Sk, H, Hkv, D, int(causal), scale, _stream()), "tt_attn_bwd")
    return dq, dk, dv


@attention_bwd.register_fake
def _(q, k, v, o, do, lse, causal, scale, row_lo=None, col_hi=None):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, row_lo=None, col_hi=None, sinks=None):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        s32 = None if sinks is None else sinks.detach().float().contiguous()
        o, lse = torch.ops.tt_b200.attention_fwd(q, k, v, causal, scale, row_lo, s32)
        ctx.save_for_backward(q, k, v, o, lse, row_lo, col_hi, sinks)
        ctx.causal, ctx.scale = causal, scale
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse, row_lo, col_hi, sinks = ctx.saved_tensors
        do = do.contiguous()
        dq, dk, dv = torch.ops.tt_b200.attention_bwd(q, k, v, o, do, lse, ctx.causal, ctx.scale, row_lo, col_hi)
        dsinks = None
        if sinks is not None and ctx.needs_input_grad[7]:
            # the sink has probability exp(sink - lse) and no value: d sink = - sum_i p_sink,i * (dO_i . O_i)
            delta = (do.float() * o.float()).sum(-1).transpose(1, 2)                     # [B,H,S]
            p_sink = torch.exp(sinks.float().view(1, -1, 1) - lse)
            dsinks = -(p_sink * delta).sum((0, 2)).to(sinks.dtype)
        return dq, dk, dv, None, None, None, None, dsinks


def range_bounds(doc_ids: Tensor | None, window: int | None, B: int, S: int, device) -> tuple[Tensor, Tensor]:
    """Per-query first visible key and per-key last visible query (int32 [B, S]) of a causal mask restricted to the
    token's own document (a document is a maximal run of equal ids) and/or to a sliding window."""
    idx = torch.arange(S, device=device, dtype=torch.int32).expand(B, S)
    if doc_ids is not None:
        d = doc_ids.to(device)
        edge = d[:, 1:] != d[:, :-1]
        one = torch.ones((B, 1), dtype=torch.bool, device=device)
        starts = torch.where(torch.cat((one, edge), 1), idx, torch.zeros_like(idx))
        lo = torch.cummax(starts, dim=1).values
        ends = torch.where(torch.cat((edge, one), 1), idx, torch.full_like(idx, S - 1))
        hi = torch.flip(torch.cummin(torch.flip(ends, (1,)), dim=1).values, (1,))
    else:
        lo, hi = torch.zeros_like(idx), torch.full_like(idx, S - 1)
    if window is not None:
        lo = torch.maximum(lo, idx - (window - 1))
        hi = torch.minimum(hi, idx + (window - 1))
    return lo.to(torch.int32).contiguous(), hi.to(torch.int32).contiguous()


def attention_supported(q: Tensor, k: Tensor, v: Tensor | None = None) -> bool:
    B, Sq, H, D = q.shape
    Dv = D if v is None else v.shape[-1]
    if q.dtype != torch.bfloat16:
        return False
    L = _lib()
    if D == 128 and Dv == 128:
        return L.tt_attn_supported(Sq, k.shape[1], H, k.shape[2], D) == 0
    return (hasattr(L, "tt_attn_supported_dims") and hasattr(L, "tt_attn_bwd_dims")
            and L.tt_attn_supported_dims(Sq, k.shape[1], H, k.shape[2], D, Dv) == 0)


def attention(q, k, v, *, causal=True, scale=None, window=None, doc_ids=None, sinks=None, return_lse=False):
    """Flash attention kernel for causal / full attention and for causal attention restricted to documents and/or a
    sliding window (contiguous key ranges), with optional per-head attention sinks; unsupported shapes take the PyTorch
    definition."""
    ranged = window is not None or doc_ids is not None
    ok = k.dtype == q.dtype and v.dtype == q.dtype and attention_supported(q, k, v)
    if ok and sinks is not None:
        ok = native.has("tt_attn_fwd_sinks")
    if ok and ranged:
        ok = bool(causal) and q.shape[1] == k.shape[1]
    if ok:
        scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        if ranged:
            lo, hi = range_bounds(doc_ids, window, q.shape[0], q.shape[1], q.device)
            o, lse = _AttnFn.apply(q, k, v, True, scale, lo, hi, sinks)
        else:
            o, lse = _AttnFn.apply(q, k, v, bool(causal), scale, None, None, sinks)
        return (o, lse) if return_lse else o
    warn_once(logger, f"attention shape/mask q={tuple(q.shape)} k={tuple(k.shape)} dtype={q.dtype} "
                      f"window={window} doc={doc_ids is not None} sinks={sinks is not None} takes the PyTorch path")
    return ref.attention(q, k, v, causal=causal, scale=scale, window=window, doc_ids=doc_ids, sinks=sinks, return_lse=return_lse)


# =============================================================================== cross entropy
@torch.library.custom_op("tt_b200::ce_fwd", mutates_args=())
def ce_fwd(logits: Tensor, labels: Tensor, ignore_index: int) -> tuple[Tensor, Tensor, Tensor]:
    """Returns (loss_sum [], lse [rows], per-row log-prob of the label [rows])."""
    rows, V = logits.shape
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    loss_rows = torch.empty(rows, dtype=torch.float32, device=logits.device)
    logprob = torch.empty(rows, dtype=torch.float32, device=logits.device)
    loss = torch.zeros((), dtype=torch.float32, device=logits.device)
    _ck(_lib().tt_ce_fwd(logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), loss_rows.data_ptr(), logprob.data_ptr(),
                         loss.data_ptr(), rows, V, logits.stride(0), ignore_index, _dt(logits), _stream()), "tt_ce_fwd")
    return loss, lse, logprob


@ce_fwd.register_fake
def _(logits, labels, ignore_index):
    r = logits.shape[0]
    return logits.new_empty((), dtype=torch.float32), logits.new_empty(r, dtype=torch.float32), logits.new_empty(r, dtype=torch.float32)


@torch.library.custom_op("tt_b200::ce_bwd", mutates_args=())
def ce_bwd(logits: Tensor, labels: Tensor, lse: Tensor, gscale: Tensor | None, row_scale: Tensor | None,
           ignore_index: int, negate: bool) -> Tensor:
    rows, V = logits.shape
    d = torch.empty_like(logits)
    _ck(_lib().tt_ce_bwd(logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), _p(gscale), _p(row_scale), d.data_ptr(), rows,
                         V, logits.stride(0), ignore_index, int(negate), _dt(logits), _stream()), "tt_ce_bwd")
    return d


@ce_bwd.register_fake
def _(logits, labels, lse, gscale, row_scale, ignore_index, negate):
    return torch.empty_like(logits)


class _CESumFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits2d, labels, ignore_index):
        loss, lse, _ = torch.ops.tt_b200.ce_fwd(logits2d, labels, ignore_index)
        ctx.save_for_backward(logits2d, labels, lse)
        ctx.ignore_index = ignore_index
        return loss

    @staticmethod
    def backward(ctx, g):
        logits2d, labels, lse = ctx.saved_tensors
        gs = g.to(torch.float32).reshape(1).contiguous()
        return torch.ops.tt_b200.ce_bwd(logits2d, labels, lse, gs, None, ctx.ignore_index, False), None, None


def _ce_ready(logits: Tensor) -> Tensor | None:
    if logits.dtype not in (torch.bfloat16, torch.float32):
        return None
    l2 = logits.reshape(-1, logits.shape[-1])
    if l2.stride(-1) != 1 or l2.stride(0) % 8:
        l2 = l2.contiguous()
        if l2.stride(0) % 8:
            return None
    return l2


def cross_entropy_sum(logits: Tensor, labels: Tensor, ignore_index: int = -100) -> Tensor:
    l2 = _ce_ready(logits)
    if l2 is None:
        return ref.cross_entropy_sum(logits, labels, ignore_index)
    return _CESumFn.apply(l2, labels.reshape(-1).to(torch.int64).contiguous(), ignore_index)


class _LogprobFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits2d, labels):
        _, lse, lp = torch.ops.tt_b200.ce_fwd(logits2d, labels, -(2**31))
        ctx.save_for_backward(logits2d, labels, lse)
        return lp

    @staticmethod
    def backward(ctx, g):
        logits2d, labels, lse = ctx.saved_tensors
        # d logprob / d logits = onehot - softmax = -(softmax - onehot)
        return torch.ops.tt_b200.ce_bwd(logits2d, labels, lse, None, g.to(torch.float32).contiguous(), -(2**31), True), None


def token_logprobs(logits: Tensor, labels: Tensor) -> Tensor:
    l2 = _ce_ready(logits)
    if l2 is None:
        return ref.token_logprobs(logits, labels)
    return _LogprobFn.apply(l2, labels.reshape(-1).to(torch.int64).contiguous()).view(labels.shape)


# =============================================================================== optimizer
_scratch: dict = {}


def _scratch_buf(device, n: int) -> Tensor:
    key = (device, n)
    if key not in _scratch:
        _scratch[key] = torch.empty(n, dtype=torch.float32, device=device)
    return _scratch[key]


def adamw_flat(param, grad, exp_avg, exp_avg_sq, shadow, *, lr, beta1, beta2, eps, weight_decay, step, decoupled=True,
               grad_scale=None):
    assert param.dtype == torch.float32 and grad.dtype == torch.float32
    _MX_CACHE.clear()      # the kernel rewrites compute copies of the weights in place, behind the version counters
    if shadow is not None:
        assert shadow.dtype == torch.bfloat16 and shadow.numel() == param.numel()
    gs = None
    if grad_scale is not None:
        gs = grad_scale if torch.is_tensor(grad_scale) else torch.tensor(float(grad_scale), device=param.device)
        gs = gs.to(torch.float32).reshape(1)
    _ck(_lib().tt_adamw(param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), _p(shadow),
                        param.numel(), lr, beta1, beta2, eps, weight_decay, int(step), int(decoupled), _p(gs), _stream()),
        "tt_adamw")


def sumsq(flat: Tensor, out: Tensor | None = None, accumulate: bool = False) -> Tensor:
    if out is None:
        out = torch.empty((), dtype=torch.float32, device=flat.device)
    scratch = _scratch_buf(flat.device, 2048)
    _ck(_lib().tt_sumsq(flat.data_ptr(), scratch.data_ptr(), out.data_ptr(), flat.numel(), _dt(flat), int(accumulate), _stream()),
        "tt_sumsq")
    return out


# =============================================================================== MoE (see csrc/moe.cu)
class _RouteFn(torch.autograd.Function):
    """scores -> top-k -> (normalised, scaled) weights + histogram, one warp per token (``csrc/moe.cu``)."""

    @staticmethod
    def forward(ctx, logits, expert_bias, top_k, softmax, norm, scale):
        T, E = logits.shape
        top = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
        idx = torch.empty(T, top_k, dtype=torch.int64, device=logits.device)
        counts = torch.zeros(E, dtype=torch.float32, device=logits.device)
        _ck(_lib().tt_moe_route_fwd(logits.data_ptr(), _p(expert_bias), top.data_ptr(), idx.data_ptr(), counts.data_ptr(), T, E,
                                    top_k, int(softmax), int(norm), float(scale), _stream()), "tt_moe_route_fwd")
        ctx.save_for_backward(logits, idx)
        ctx.cfg = (top_k, softmax, norm, scale)
        ctx.mark_non_differentiable(idx, counts)
        return top, idx, counts

    @staticmethod
    def backward(ctx, gtop, _gi, _gc):
        logits, idx = ctx.saved_tensors
        top_k, softmax, norm, scale = ctx.cfg
        T, E = logits.shape
        gl = torch.empty_like(logits)
        _ck(_lib().tt_moe_route_bwd(logits.data_ptr(), idx.data_ptr(), gtop.contiguous().float().data_ptr(), gl.data_ptr(), T, E,
                                    top_k, int(softmax), int(norm), float(scale), _stream()), "tt_moe_route_bwd")
        return gl, None, None, None, None, None


def moe_route(x, gate_w, gate_b, expert_bias, *, top_k, score_func, route_norm, route_scale, num_expert_groups=None,
              num_limited_groups=None, force_balance=False):
    E = gate_w.shape[0]
    if num_expert_groups is not None or force_balance or E > 256 or top_k > 16 or score_func not in ("softmax", "sigmoid"):
        return ref.moe_route(x, gate_w, gate_b, expert_bias, top_k=top_k, score_func=score_func, route_norm=route_norm,
                             route_scale=route_scale, num_expert_groups=num_expert_groups,
                             num_limited_groups=num_limited_groups, force_balance=force_balance)
    # the gate product stays in fp32 (library GEMM); everything after it is one kernel
    logits = torch.nn.functional.linear(x.float(), gate_w.float(), None if gate_b is None else gate_b.float()).contiguous()
    eb = None if expert_bias is None else expert_bias.float().contiguous()
    return _RouteFn.apply(logits, eb, top_k, score_func == "softmax", bool(route_norm), float(route_scale))


def moe_sort(expert_idx, num_experts: int):
    """Stable counting sort of the (token, slot) pairs by expert: (order int64 [T*k], counts int64 [E])."""
    flat = expert_idx.reshape(-1).contiguous()
    n = flat.numel()
    counts_f = torch.zeros(num_experts, dtype=torch.float32, device=flat.device)
    counts_f.index_add_(0, flat, torch.ones(n, dtype=torch.float32, device=flat.device))
    order = torch.empty(n, dtype=torch.int64, device=flat.device)
    counts = torch.empty(num_experts, dtype=torch.int64, device=flat.device)
    _ck(_lib().tt_moe_sort(flat.data_ptr(), counts_f.data_ptr(), order.data_ptr(), counts.data_ptr(), n, num_experts, _stream()),
        "tt_moe_sort")
    return order, counts


class _GatherSrc(torch.autograd.Function):
    """out[j] = x[src[j]] (zero row where src < 0); backward sums the k copies of each token through ``pos``."""

    @staticmethod
    def forward(ctx, x, src, pos, top_k):
        R, D = src.numel(), x.shape[-1]
        out = torch.empty(R, D, dtype=x.dtype, device=x.device)
        _ck(_lib().tt_moe_gather(x.data_ptr(), src.data_ptr(), None, out.data_ptr(), R, D, _stream()), "tt_moe_gather")
        ctx.save_for_backward(pos)
        ctx.shape, ctx.k = x.shape, top_k
        return out

    @staticmethod
    def backward(ctx, g):
        (pos,) = ctx.saved_tensors
        T, D = ctx.shape
        gx = torch.empty(T, D, dtype=g.dtype, device=g.device)
        _ck(_lib().tt_moe_combine(g.contiguous().data_ptr(), pos.data_ptr(), None, gx.data_ptr(), T, ctx.k, D, _stream()),
            "tt_moe_combine")
        return gx, None, None, None


class _CombinePos(torch.autograd.Function):
    """out[t] = sum_s w[t,s] * rows[pos[t,s]] in fp32; ``pair`` [R] is the inverse map (flat pair index per row, -1 = padding)."""

    @staticmethod
    def forward(ctx, rows, pos, pair, w, T, top_k):
        D = rows.shape[-1]
        out = torch.empty(T, D, dtype=rows.dtype, device=rows.device)
        wf = None if w is None else w.float().contiguous()
        _ck(_lib().tt_moe_combine(rows.data_ptr(), pos.data_ptr(), _p(wf), out.data_ptr(), T, top_k, D, _stream()), "tt_moe_combine")
        ctx.save_for_backward(rows, pos, pair, wf if wf is not None else torch.empty(0, device=rows.device))
        ctx.has_w, ctx.k = w is not None, top_k
        return out

    @staticmethod
    def backward(ctx, g):
        rows, pos, pair, wf = ctx.saved_tensors
        g = g.contiguous()
        R, D = rows.shape
        T = g.shape[0]
        src = torch.where(pair >= 0, pair // ctx.k, pair).to(torch.int32)
        scale = None
        if ctx.has_w:
            scale = torch.where(pair >= 0, wf.reshape(-1)[pair.clamp(min=0).long()], torch.zeros((), device=g.device)).contiguous()
        grows = torch.empty_like(rows)
        _ck(_lib().tt_moe_gather(g.data_ptr(), src.data_ptr(), _p(scale), grows.data_ptr(), R, D, _stream()), "tt_moe_gather")
        gw = None
        if ctx.has_w and ctx.needs_input_grad[3]:
            gw = torch.empty(T, ctx.k, dtype=torch.float32, device=g.device)
            _ck(_lib().tt_moe_rowdot(rows.data_ptr(), pos.data_ptr(), g.data_ptr(), gw.data_ptr(), T, ctx.k, D, _stream()),
                "tt_moe_rowdot")
        return grows, None, None, gw, None, None


class _ScaleRowsFn(torch.autograd.Function):
    """``out[r, :] = rows[r, :] * scale[r]`` (bf16 rows, fp32 scales, one pass). Backward: the same pass on the output
    gradient and one row-dot kernel for the scales' gradient."""

    @staticmethod
    def forward(ctx, rows, scale):
        R, D = rows.shape
        out = torch.empty_like(rows)
        _ck(_lib().tt_moe_gather(rows.data_ptr(), None, scale.data_ptr(), out.data_ptr(), R, D, _stream()), "tt_moe_gather(scale)")
        ctx.save_for_backward(rows, scale)
        return out

    @staticmethod
    def backward(ctx, g):
        rows, scale = ctx.saved_tensors
        R, D = rows.shape
        g = g.contiguous()
        g_rows = g_scale = None
        if ctx.needs_input_grad[0]:
            g_rows = torch.empty_like(rows)
            _ck(_lib().tt_moe_gather(g.data_ptr(), None, scale.data_ptr(), g_rows.data_ptr(), R, D, _stream()), "tt_moe_gather(scale)")
        if ctx.needs_input_grad[1]:
            g_scale = torch.empty(R, dtype=torch.float32, device=rows.device)
            _ck(_lib().tt_moe_rowdot(rows.data_ptr(), None, g.data_ptr(), g_scale.data_ptr(), R, 1, D, _stream()), "tt_moe_rowdot")
        return g_rows, g_scale


def scale_rows(rows: Tensor, scale: Tensor) -> Tensor:
    """Rows times one fp32 factor each. bf16 rows of a multiple of 8 elements take the fused kernels."""
    if rows.is_cuda and rows.dtype == torch.bfloat16 and rows.dim() == 2 and rows.shape[1] % 8 == 0 and rows.is_contiguous():
        return _ScaleRowsFn.apply(rows, scale.reshape(-1).to(torch.float32).contiguous())
    return (rows.float() * scale.reshape(-1, 1)).to(rows.dtype)


def moe_gather_src(x, src, pos, top_k: int):
    return _GatherSrc.apply(x.contiguous(), src, pos, top_k)


def moe_combine_pos(rows, pos, pair, weights, num_tokens: int, top_k: int):
    return _CombinePos.apply(rows.contiguous(), pos, pair, weights, num_tokens, top_k)


def inverse_positions(order: Tensor) -> Tensor:
    """``pos`` with ``pos[order[j]] = j`` (int32): where each (token, slot) pair sits in the expert-sorted order."""
    n = order.numel()
    return torch.empty(n, dtype=torch.int32, device=order.device).index_copy_(
        0, order, torch.arange(n, dtype=torch.int32, device=order.device))


def _rows_kernel_ok(x: Tensor) -> bool:
    return x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[-1] % 8 == 0


def copy_rows_where(rows: Tensor, keep: Tensor) -> Tensor:
    """A copy of ``rows`` [R, D] with the rows where ``keep`` [R] is false set to zero, in one vectorised pass (also the
    copy out of a communication buffer that the next exchange overwrites)."""
    R = rows.shape[0]
    if not (_rows_kernel_ok(rows) and rows.is_contiguous()):
        return torch.where(keep.unsqueeze(1), rows, torch.zeros((), dtype=rows.dtype, device=rows.device))
    src = torch.where(keep, torch.arange(R, dtype=torch.int32, device=rows.device), torch.full((), -1, dtype=torch.int32, device=rows.device))
    out = torch.empty_like(rows)
    _ck(_lib().tt_moe_gather(rows.data_ptr(), src.data_ptr(), None, out.data_ptr(), R, rows.shape[1], _stream()), "tt_moe_gather(copy)")
    return out


def sum_copies(rows: Tensor, pos: Tensor, num_tokens: int, top_k: int) -> Tensor:
    """``out[t] = sum_s rows[pos[t * k + s]]``: the gradient of a token from the gradients of its k routed copies."""
    out = torch.empty(num_tokens, rows.shape[-1], dtype=rows.dtype, device=rows.device)
    _ck(_lib().tt_moe_combine(rows.contiguous().data_ptr(), pos.data_ptr(), None, out.data_ptr(), num_tokens, top_k, rows.shape[-1],
                              _stream()), "tt_moe_combine")
    return out


def moe_gather_rows(x, order, top_k: int):
    if _rows_kernel_ok(x) and order.numel() == x.shape[0] * top_k:
        return _GatherSrc.apply(x.contiguous(), (order // top_k).to(torch.int32), inverse_positions(order), top_k)
    return x[order // top_k]


def moe_scatter_combine(rows, order, weights, num_tokens: int, top_k: int):
    n = order.numel()
    if _rows_kernel_ok(rows) and n == num_tokens * top_k:
        # one pass: every token reads its k rows through the inverse of the sort and sums them (weighted) in fp32
        return _CombinePos.apply(rows[:n].contiguous(), inverse_positions(order), order, weights, num_tokens, top_k)
    D = rows.shape[-1]
    unsorted = rows.new_zeros(num_tokens * top_k, D)
    unsorted[order] = rows[: order.numel()]
    unsorted = unsorted.view(num_tokens, top_k, D)
    if weights is None:
        return unsorted.sum(dim=1)
    return torch.bmm(weights.reshape(-1, 1, top_k), unsorted.float()).to(rows.dtype).squeeze(1)


class _GroupedLinearFn(torch.autograd.Function):
    """Per-expert GEMMs launched back to back on the tcgen05 kernel; group sizes are read once
    per call (one small device-to-host copy shared by the three expert GEMMs of a layer)."""

    @staticmethod
    def forward(ctx, x, w, counts):
        sizes = _group_sizes(counts)
        out = x.new_zeros(x.shape[0], w.shape[1])
        s = 0
        for e, n in enumerate(sizes):
            if n:
                gemm_into(x[s : s + n], w[e], out[s : s + n])
            s += n
        ctx.save_for_backward(x, w)
        ctx.sizes = sizes
        return out

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        gy = gy.contiguous()
        gx = torch.zeros_like(x)
        gw = torch.zeros_like(w)
        s = 0
        for e, n in enumerate(ctx.sizes):
            if n:
                gemm_into(gy[s : s + n], w[e], gx[s : s + n], b_mn=True)
                gemm_into(gy[s : s + n], x[s : s + n], gw[e], a_mn=True, b_mn=True)
            s += n
        return gx, gw, None


_sizes_cache: dict = {}


def _group_sizes(counts: Tensor) -> list[int]:
    key = (counts.data_ptr(), counts._version)
    hit = _sizes_cache.get("k")
    if hit is not None and hit[0] == key:
        return hit[1]
    sizes = [int(v) for v in counts.tolist()]
    _sizes_cache["k"] = (key, sizes)
    return sizes


class _GroupedGemmFn(torch.autograd.Function):
    """One launch per GEMM over all experts; group boundaries stay on the device (``csrc/grouped_gemm.cu``).
    Needs every group size to be a multiple of 64 (the dispatcher pads with zero rows)."""

    @staticmethod
    def forward(ctx, x, w, offs):
        R, K = x.shape
        E, N, _ = w.shape
        y = x.new_zeros(R, N)
        _ck(_lib().tt_grouped_gemm(x.data_ptr(), w.data_ptr(), y.data_ptr(), offs.data_ptr(), R, E, N, K, 0, x.stride(0),
                                   y.stride(0), _stream()), "tt_grouped_gemm")
        ctx.save_for_backward(x, w, offs)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w, offs = ctx.saved_tensors
        gy = gy.contiguous()
        R, K = x.shape
        E, N, _ = w.shape
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = torch.zeros_like(x)
            # w viewed as [E, K' = N, N' = K]: the contraction runs over w's first matrix dimension (b_mn)
            _ck(_lib().tt_grouped_gemm(gy.data_ptr(), w.data_ptr(), gx.data_ptr(), offs.data_ptr(), R, E, K, N, 1, gy.stride(0),
                                       gx.stride(0), _stream()), "tt_grouped_gemm(dgrad)")
        if ctx.needs_input_grad[1]:
            gw = torch.zeros_like(w)
            _ck(_lib().tt_grouped_gemm_wgrad(gy.data_ptr(), x.data_ptr(), gw.data_ptr(), offs.data_ptr(), R, E, N, K,
                                             gy.stride(0), x.stride(0), int(gw.dtype == torch.float32), _stream()),
                "tt_grouped_gemm_wgrad")
        return gx, gw, None


def grouped_linear(x, w, counts):
    ok = x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w.shape[1] % 8 == 0
    aligned = getattr(counts, "_tt_aligned", 0)
    if ok and aligned and aligned % 64 == 0 and w.shape[1] % 64 == 0 and w.shape[2] % 64 == 0 and native.has("tt_grouped_gemm"):
        offs = torch.cumsum(counts, 0).to(torch.int32)
        return _GroupedGemmFn.apply(x.contiguous(), w.contiguous(), offs)
    if ok:
        return _GroupedLinearFn.apply(x.contiguous(), w, counts)
    from .moe_ops import _GroupedLinearRef

    return _GroupedLinearRef.apply(x, w, counts)


# =============================================================================== generation (see csrc/serving.cu)
def kv_write(k_cache: Tensor, v_cache: Tensor, k: Tensor, v: Tensor, slots: Tensor) -> None:
    T, Hkv, D = k.shape
    if k.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or D != 128:
        kc, vc = k_cache.view(-1, Hkv, D), v_cache.view(-1, Hkv, D)
        kc.index_copy_(0, slots.long(), k.to(kc.dtype))
        vc.index_copy_(0, slots.long(), v.to(vc.dtype))
        return
    k, v = k.contiguous(), v.contiguous()
    _ck(_lib().tt_kv_write(k_cache.data_ptr(), v_cache.data_ptr(), k.data_ptr(), v.data_ptr(), slots.to(torch.int32).data_ptr(),
                           T, Hkv, D, _stream()), "tt_kv_write")


def paged_decode(q: Tensor, k_cache: Tensor, v_cache: Tensor, block_tables: Tensor, context_lens: Tensor, scale: float) -> Tensor:
    B, H, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or D != 128 or (H // Hkv) not in (1, 2, 4, 8):
        raise NotImplementedError(f"paged decode kernel: bf16, head_dim 128 and 1/2/4/8 query heads per kv head (got {q.dtype}, {D}, {H}/{Hkv})")
    q = q.contiguous()
    out = torch.empty_like(q)
    bt = block_tables if block_tables.dtype == torch.int32 else block_tables.to(torch.int32)
    cl = context_lens if context_lens.dtype == torch.int32 else context_lens.to(torch.int32)
    _ck(_lib().tt_paged_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), bt.contiguous().data_ptr(), cl.data_ptr(),
                               out.data_ptr(), float(scale), B, H, Hkv, D, bs, bt.shape[1], _stream()), "tt_paged_decode")
    return out


def sample(logits: Tensor, temperature: float, uniforms: Tensor, top_p: float = 1.0) -> tuple[Tensor, Tensor]:
    """Greedy (temperature <= 0) or index-order multinomial / nucleus sampling; one CTA per row."""
    B, V = logits.shape
    if logits.dtype not in (torch.float32, torch.bfloat16):
        logits = logits.float()
    if logits.stride(-1) != 1:
        logits = logits.contiguous()
    tok = torch.empty(B, dtype=torch.int64, device=logits.device)
    lp = torch.empty(B, dtype=torch.float32, device=logits.device)
    u = uniforms.to(torch.float32).contiguous()
    if top_p < 1.0 and temperature > 0.0:
        _ck(_lib().tt_sample_top_p(logits.data_ptr(), u.data_ptr(), tok.data_ptr(), lp.data_ptr(), B, V, logits.stride(0),
                                   float(temperature), float(top_p), int(logits.dtype == torch.bfloat16), _stream()),
            "tt_sample_top_p")
        return tok, lp
    _ck(_lib().tt_sample(logits.data_ptr(), u.data_ptr(), tok.data_ptr(), lp.data_ptr(), B, V, logits.stride(0), float(temperature),
                         int(logits.dtype == torch.bfloat16), _stream()), "tt_sample")
    return tok, lp


# =============================================================================== float8 GEMM (csrc/gemm.cu, kind::f8f6f4)
def quantize_fp8_operand(x: Tensor, rowwise: bool, dtype=torch.float8_e4m3fn):
    """Quantise a 2-D bf16 GEMM operand ``x`` [R, K] along its last (contraction) dimension with the native kernels and
    return (q [R, K] contiguous, scale): one scale per row (power of two) when ``rowwise`` else one per tensor.
    ``x`` may be a transposed view of a row-major matrix: then the transposing kernels are used, so no copy of the
    high-precision operand is made. Returns None when the layout or shape is not covered."""
    if x.dim() != 2 or x.dtype != torch.bfloat16 or not native.has("tt_fp8_quant_rows"):
        return None
    R, K = x.shape
    e5m2 = int(dtype == torch.float8_e5m2)
    L = _lib()
    q = torch.empty(R, K, dtype=dtype, device=x.device)
    if x.stride(1) == 1 and x.stride(0) % 8 == 0 and K % 8 == 0 and x.data_ptr() % 16 == 0:
        if rowwise:
            scale = torch.empty(R, dtype=torch.float32, device=x.device)
            _ck(L.tt_fp8_quant_rows(x.data_ptr(), x.stride(0), R, K, q.data_ptr(), scale.data_ptr(), e5m2, 1, _stream()),
                "tt_fp8_quant_rows")
        else:
            scale = torch.empty(1, dtype=torch.float32, device=x.device)
            _ck(L.tt_fp8_quant_tensor(x.data_ptr(), x.stride(0), R, K, q.data_ptr(), scale.data_ptr(), 0, e5m2, _stream()),
                "tt_fp8_quant_tensor")
        return q, scale
    if x.stride(0) == 1 and x.stride(1) % 8 == 0 and R % 8 == 0 and K % 16 == 0 and x.data_ptr() % 16 == 0:
        # x = m^T for the row-major m [K, R]: contraction runs down the columns of m
        if rowwise:
            scale = torch.empty(R, dtype=torch.float32, device=x.device)
            _ck(L.tt_fp8_quant_cols(x.data_ptr(), x.stride(1), K, R, q.data_ptr(), scale.data_ptr(), e5m2, 1, _stream()),
                "tt_fp8_quant_cols")
        else:
            scale = torch.empty(1, dtype=torch.float32, device=x.device)
            _ck(L.tt_fp8_quant_tensor(x.data_ptr(), x.stride(1), K, R, q.data_ptr(), scale.data_ptr(), 1, e5m2, _stream()),
                "tt_fp8_quant_tensor")
        return q, scale
    return None


def quantize_mxfp8_operand(x: Tensor):
    """MXFP8-quantise a 2-D bf16 GEMM operand ``x`` [R, K] along K (blocks of 32): returns (e4m3 [R, K] contiguous,
    uint8 E8M0 scales [R, K/32]) or None when the layout is not covered. A transposed view of a row-major matrix goes
    through the transposing kernel (no high-precision copy)."""
    if x.dim() != 2 or x.dtype != torch.bfloat16 or not native.has("tt_mxfp8_quant_rows"):
        return None
    R, K = x.shape
    if K % 32 or x.data_ptr() % 16:
        return None
    L = _lib()
    q = torch.empty(R, K, dtype=torch.float8_e4m3fn, device=x.device)
    sc = torch.empty(R, K // 32, dtype=torch.uint8, device=x.device)
    if x.stride(1) == 1 and x.stride(0) % 8 == 0:
        _ck(L.tt_mxfp8_quant_rows(x.data_ptr(), x.stride(0), R, K, q.data_ptr(), sc.data_ptr(), _stream()), "tt_mxfp8_quant_rows")
        return q, sc
    if x.stride(0) == 1 and x.stride(1) % 8 == 0 and R % 8 == 0:
        _ck(L.tt_mxfp8_quant_cols(x.data_ptr(), x.stride(1), K, R, q.data_ptr(), sc.data_ptr(), _stream()), "tt_mxfp8_quant_cols")
        return q, sc
    return None


# ---- MXFP8 linear algebra as one dispatcher-visible op ------------------------------------------------------------
# Recently quantised operands, keyed by the source's address, layout and version. The entry keeps the source tensor alive,
# so its address cannot be handed to another tensor while the entry exists; an in-place write bumps the version. Serves
# the activations that several linears share (wq / wk / wv, w1 / w3 and their weight-gradient GEMMs).
_MX_CACHE: list = []
_MX_CACHE_SIZE = 3


def _mx_operand(x: Tensor, transposed: bool):
    """MXFP8 operand of a GEMM whose contraction runs along the last dimension of ``x`` (or of ``x.t()`` when
    ``transposed``): (e4m3 [R, K] contiguous, E8M0 scales in the block-scaled MMA's layout), or None when the layout is
    not covered by the native kernels."""
    key = (x.data_ptr(), tuple(x.shape), tuple(x.stride()), x._version, transposed)
    for i, (k, _, out) in enumerate(_MX_CACHE):
        if k == key:
            _MX_CACHE.append(_MX_CACHE.pop(i))
            return out
    L = _lib()
    if x.dim() != 2 or x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        return None
    rows, cols = x.shape
    if transposed:        # operand = x^T [cols, rows], contraction along x's rows
        R, K = cols, rows
        if K % 32 or R % 8:
            return None
    else:
        R, K = rows, cols
        if K % 32:
            return None
    q = torch.empty(R, K, dtype=torch.float8_e4m3fn, device=x.device)
    sc = torch.empty(L.tt_mx_scales_bytes(R, 256, K), dtype=torch.uint8, device=x.device)
    if R % 256 or (K // 32) % 4:
        sc.fill_(127)     # rows / K blocks past the end carry the neutral scale 2^0 (their data is zero-filled by TMA)
    if transposed:
        _ck(L.tt_mxfp8_quant_cols_swz(x.data_ptr(), x.stride(0), rows, cols, q.data_ptr(), sc.data_ptr(), _stream()),
            "tt_mxfp8_quant_cols_swz")
    else:
        _ck(L.tt_mxfp8_quant_rows_swz(x.data_ptr(), x.stride(0), rows, cols, q.data_ptr(), sc.data_ptr(), _stream()),
            "tt_mxfp8_quant_rows_swz")
    out = (q, sc)
    _MX_CACHE.append((key, x, out))
    if len(_MX_CACHE) > _MX_CACHE_SIZE:
        _MX_CACHE.pop(0)
    return out


def mx_cache_clear() -> None:
    _MX_CACHE.clear()


def _mx_mm_into(a: Tensor, b: Tensor, a_t: bool, b_t: bool, out: Tensor) -> bool:
    """``out = op(a) @ op(b)^T`` with both operands MXFP8-quantised along the contraction; False when a layout is not
    covered (the caller then uses the PyTorch definition)."""
    qa, qb = _mx_operand(a, a_t), _mx_operand(b, b_t)
    if qa is None or qb is None or out.stride(1) != 1:
        return False
    (A, sa), (B, sb) = qa, qb
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K and out.shape == (M, N)
    _ck(_lib().tt_gemm_mxfp8(A.data_ptr(), B.data_ptr(), sa.data_ptr(), sb.data_ptr(), out.data_ptr(), M, N, K, A.stride(0),
                             B.stride(0), out.stride(0), int(out.dtype == torch.float32), _stream()), "tt_gemm_mxfp8")
    return True


@torch.library.custom_op("tt_b200::mx_mm", mutates_args=())
def mx_mm(a: Tensor, b: Tensor, a_t: bool, b_t: bool, out_fp32: bool) -> Tensor:
    """``op(a) [M,K] @ op(b) [N,K]^T`` (``op`` = transpose when the flag is set) with MXFP8 operands: both are quantised
    here (e4m3 data, one E8M0 scale per 32 elements of K, RCEIL) and multiplied by the block-scaled tensor-core kernel.
    One op, so per-op activation checkpointing can keep its output like any other matmul."""
    M = a.shape[1] if a_t else a.shape[0]
    N = b.shape[1] if b_t else b.shape[0]
    out = torch.empty((M, N), dtype=torch.float32 if out_fp32 else torch.bfloat16, device=a.device)
    if not _mx_mm_into(a, b, a_t, b_t, out):
        from .quant import _mx_mm

        out.copy_(_mx_mm(a.t() if a_t else a, b.t() if b_t else b, out.dtype))
    return out


@mx_mm.register_fake
def _(a, b, a_t, b_t, out_fp32):
    M = a.shape[1] if a_t else a.shape[0]
    N = b.shape[1] if b_t else b.shape[0]
    return a.new_empty((M, N), dtype=torch.float32 if out_fp32 else torch.bfloat16)


class _MxLinearFn(torch.autograd.Function):
    """MXFP8 linear: forward ``x W^T``, input gradient ``dy W`` (W quantised down its columns) and weight gradient
    ``dy^T x`` (both quantised down their rows, i.e. along the tokens), each through ``tt_b200::mx_mm``. The weight
    gradient goes straight into the FSDP unit's gradient buffer when the weight carries a slot."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = _rows2d(x)
        y = torch.ops.tt_b200.mx_mm(x2, w, False, False, False)
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        ctx.grad_slot = getattr(w, "_grad_slot", None)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = _rows2d(gy)
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = torch.ops.tt_b200.mx_mm(g2, w, False, True, False).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            slot = ctx.grad_slot
            if slot is not None:
                if not slot.begin() and _mx_mm_into(g2, x2, True, True, slot.tensor):
                    pass                                            # first gradient of this backward: written in place
                else:
                    slot.tensor.add_(torch.ops.tt_b200.mx_mm(g2, x2, True, True, True))
                gw = _placeholder(w)
            else:
                gw = torch.ops.tt_b200.mx_mm(g2, x2, True, True, False)
        return gx, gw


def mx_linear(x: Tensor, weight: Tensor) -> Tensor | None:
    """The native MXFP8 linear, or None when dtype / shape / library do not allow it."""
    if not (x.is_cuda and native.has("tt_mxfp8_quant_rows_swz") and native.has("tt_gemm_mxfp8")):
        return None
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.dim() != 2 or weight.stride(1) != 1:
        return None
    K, N = x.shape[-1], weight.shape[0]
    rows = x.numel() // max(K, 1)
    if K % 32 or N % 32 or rows % 32 or weight.stride(0) % 8 or weight.data_ptr() % 16:
        return None
    return _MxLinearFn.apply(x, weight)


def _mx_grouped_launch(A, sa, B, sb, out, offs, mode: int, G: int, M: int, N: int, K: int, b_row_stride: int, b_k_stride: int):
    _ck(_lib().tt_grouped_gemm_mxfp8(A.data_ptr(), B.data_ptr(), sa.data_ptr(), sb.data_ptr(), out.data_ptr(), offs.data_ptr(),
                                     mode, G, M, N, K, A.shape[0], A.shape[1], B.shape[0], B.shape[1], b_row_stride, b_k_stride,
                                     out.stride(-2), int(out.dtype == torch.float32), _stream()), "tt_grouped_gemm_mxfp8")


class _MxGroupedFn(torch.autograd.Function):
    """Routed-expert linear ``y[r] = x[r] @ w[g(r)]^T`` in MXFP8, one launch per GEMM over all experts with the group
    boundaries read on the device (``csrc/gemm_mx.cu``, grouped form). Operands are quantised along the contraction of
    each of the three GEMMs: forward ``x`` and ``w`` along K; input gradient ``dy`` along N and ``w`` down its rows
    (one transposing pass over the weights viewed as [G * N, K]); weight gradient ``dy`` and ``x`` down their rows, so
    the 32-element blocks run along the tokens of one expert (groups start at multiples of 128 rows)."""

    @staticmethod
    def forward(ctx, x, w, offs):
        G, N, K = w.shape
        R = x.shape[0]
        (xq, xs), (wq, ws) = _mx_operand(x, False), _mx_operand(w.view(G * N, K), False)
        y = x.new_zeros(R, N)
        _mx_grouped_launch(xq, xs, wq, ws, y, offs, 0, G, R, N, K, N, 0)
        ctx.save_for_backward(x, w, offs)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w, offs = ctx.saved_tensors
        G, N, K = w.shape
        R = x.shape[0]
        gy = gy.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            (gq, gs), (wtq, wts) = _mx_operand(gy, False), _mx_operand(w.view(G * N, K), True)      # w^T: [K, G * N]
            gx = torch.zeros_like(x)
            _mx_grouped_launch(gq, gs, wtq, wts, gx, offs, 0, G, R, K, N, 0, N)
        if ctx.needs_input_grad[1]:
            (gtq, gts), (xtq, xts) = _mx_operand(gy, True), _mx_operand(x, True)                   # [N, R], [K, R]
            gw = torch.zeros_like(w)
            _mx_grouped_launch(gtq, gts, xtq, xts, gw, offs, 1, G, N, K, 128, 0, 0)
        return gx, gw, None


def mx_grouped_linear(x: Tensor, w: Tensor, counts: Tensor) -> Tensor | None:
    """The native grouped MXFP8 linear, or None when alignment / shapes / library do not allow it: bf16 operands, every
    group a multiple of 128 rows (``counts`` carries the dispatcher's alignment), N and K multiples of 128."""
    if not (x.is_cuda and native.has("tt_grouped_gemm_mxfp8") and native.has("tt_mxfp8_quant_cols_swz")):
        return None
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.dim() != 3 or x.dim() != 2:
        return None
    aligned = getattr(counts, "_tt_aligned", 0)
    G, N, K = w.shape
    if not aligned or aligned % 128 or N % 128 or K % 128 or x.shape[0] % 128 or G > 1024 or x.shape[1] != K:
        return None
    offs = torch.cumsum(counts, 0).to(torch.int32)
    return _MxGroupedFn.apply(x.contiguous(), w.contiguous(), offs)


def gemm_mxfp8(qa: Tensor, qb: Tensor, sa: Tensor, sb: Tensor, out_dtype=torch.bfloat16) -> Tensor:
    """``qa [M,K] @ qb [N,K]^T`` for MXFP8 operands (e4m3 data, E8M0 scales [rows, K/32]) on the block-scaled tensor-core
    path: the scales are re-laid into the MMA's 512-byte chunks and applied by the MMA itself."""
    M, K = qa.shape
    N = qb.shape[0]
    L = _lib()
    qa, qb = qa.contiguous(), qb.contiguous()
    sa, sb = sa.contiguous(), sb.contiguous()
    swa = torch.empty(L.tt_mx_scales_bytes(M, 256, K), dtype=torch.uint8, device=qa.device)   # 256-row padding: CTA-pair tiles
    swb = torch.empty(L.tt_mx_scales_bytes(N, 256, K), dtype=torch.uint8, device=qa.device)
    _ck(L.tt_mx_swizzle_scales(sa.data_ptr(), M, K, 256, swa.data_ptr(), _stream()), "tt_mx_swizzle_scales")
    _ck(L.tt_mx_swizzle_scales(sb.data_ptr(), N, K, 256, swb.data_ptr(), _stream()), "tt_mx_swizzle_scales")
    c_fp32 = out_dtype == torch.float32
    out = torch.empty(M, N, dtype=torch.float32 if c_fp32 else torch.bfloat16, device=qa.device)
    _ck(L.tt_gemm_mxfp8(qa.data_ptr(), qb.data_ptr(), swa.data_ptr(), swb.data_ptr(), out.data_ptr(), M, N, K, qa.stride(0),
                        qb.stride(0), out.stride(0), int(c_fp32), _stream()), "tt_gemm_mxfp8")
    return out if out.dtype == out_dtype else out.to(out_dtype)


def gemm_fp8(qa: Tensor, qb: Tensor, sa: Tensor, sb: Tensor, out_dtype=torch.bfloat16) -> Tensor:
    """``(qa [M,K] @ qb [N,K]^T) * sa * sb`` with float8 operands; ``sa``/``sb`` are scalars (tensorwise) or hold one
    scale per row of ``qa`` / ``qb`` (rowwise). fp32 accumulation in TMEM, scales applied in the epilogue."""
    M, K = qa.shape
    N = qb.shape[0]
    if K % 16:
        acc = qa.float() @ qb.float().t()
        return (acc * sa.reshape(-1, 1) * sb.reshape(1, -1)).to(out_dtype)
    qa, qb = qa.contiguous(), qb.contiguous()
    mode = 1 if (sa.numel() == 1 and sb.numel() == 1) else 2
    sa = sa.reshape(-1).float().contiguous()
    sb = sb.reshape(-1).float().contiguous()
    if mode == 2:
        if sa.numel() == 1:
            sa = sa.expand(M).contiguous()
        if sb.numel() == 1:
            sb = sb.expand(N).contiguous()
    c_fp32 = out_dtype == torch.float32
    out = torch.empty(M, N, dtype=torch.float32 if c_fp32 else torch.bfloat16, device=qa.device)
    _ck(_lib().tt_gemm_fp8(qa.data_ptr(), qb.data_ptr(), out.data_ptr(), M, N, K, qa.stride(0), qb.stride(0), out.stride(0),
                           int(c_fp32), int(qa.dtype == torch.float8_e5m2), int(qb.dtype == torch.float8_e5m2), sa.data_ptr(),
                           sb.data_ptr(), mode, _stream()), "tt_gemm_fp8")
    return out if out.dtype == out_dtype else out.to(out_dtype)
