"""Low-precision training arithmetic: float8 (tensorwise / rowwise scaling) and MXFP8 (e4m3 data
with one power-of-two E8M0 scale per 32 elements along the contraction dimension, RCEIL rounding).

Behavioural contract (torchao recipes as used by torchtitan/components/quantization/float8.py:36-63
and mx.py:33-59): every GEMM of a converted layer -- forward ``y = x W^T``, input gradient
``dx = dy W`` and weight gradient ``dW = dy^T x`` -- quantises both operands dynamically along
that GEMM's own contraction dimension, multiplies in 8 bits with fp32 accumulation and rescales;
``rowwise_with_gw_hp`` keeps the weight-gradient GEMM in bf16. Master weights stay high precision.

The functions in this file are the definition of the numerics (plain PyTorch, any device); on a
B200 the quantise + GEMM pairs run as the native block-scaled tcgen05 kernels when the library
provides them (``native.has("tt_gemm_fp8")``), otherwise the operands are dequantised and fed to the
bf16 GEMM (``emulate``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

E4M3_MAX = 448.0
E5M2_MAX = 57344.0
MX_BLOCK = 32


@dataclass(frozen=True)
class QuantRecipe:
    kind: str = "float8"          # "float8" | "mxfp8"
    scaling: str = "tensorwise"   # float8: tensorwise | rowwise | rowwise_with_gw_hp
    emulate: bool = False
    pad_token_groups: bool = True


# ---- float8 ---------------------------------------------------------------------------------
def quantize_fp8(x: torch.Tensor, axis: int | None, dtype=torch.float8_e4m3fn):
    """Returns (q, scale) with ``x ~= q.float() * scale``; ``axis`` is the contraction dimension
    (amax is taken along it, one scale per remaining row) or None for one scale per tensor.
    Rowwise scales are rounded down to a power of two, as the rowwise recipe does."""
    fmax = E4M3_MAX if dtype == torch.float8_e4m3fn else E5M2_MAX
    xf = x.float()
    if axis is None:
        amax = xf.abs().amax().clamp_min(1e-12)
        scale = amax / fmax
    else:
        amax = xf.abs().amax(dim=axis, keepdim=True).clamp_min(1e-12)
        scale = torch.exp2(torch.ceil(torch.log2(amax / fmax)))
    q = (xf / scale).clamp(-fmax, fmax).to(dtype)
    return q, scale


def _fp8_mm(a: torch.Tensor, b_t: torch.Tensor, axis_mode: str, out_dtype, grad: bool = False):
    """``a [M,K] @ b_t[N,K]^T`` with both operands quantised along K."""
    axis = None if axis_mode == "tensorwise" else -1
    a_dtype = torch.float8_e5m2 if (grad and axis_mode == "tensorwise") else torch.float8_e4m3fn
    from . import native

    if a.is_cuda and native.has("tt_gemm_fp8"):
        from .cuda_ops import gemm_fp8, quantize_fp8_operand

        # native quantisation writes operands contiguous along the contraction whatever the view's layout
        qa_sa = quantize_fp8_operand(a, axis is not None, a_dtype)
        qb_sb = quantize_fp8_operand(b_t, axis is not None, torch.float8_e4m3fn)
        qa, sa = qa_sa if qa_sa is not None else quantize_fp8(a, axis, a_dtype)
        qb, sb = qb_sb if qb_sb is not None else quantize_fp8(b_t, axis)
        return gemm_fp8(qa, qb, sa, sb, out_dtype)
    qa, sa = quantize_fp8(a, axis, a_dtype)
    qb, sb = quantize_fp8(b_t, axis)
    acc = qa.float() @ qb.float().t()
    sa2 = sa if axis is None else sa.reshape(-1, 1)
    sb2 = sb if axis is None else sb.reshape(1, -1)
    return (acc * sa2 * sb2).to(out_dtype)


class _Fp8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, recipe: QuantRecipe):
        ctx.save_for_backward(x, w)
        ctx.recipe = recipe
        mode = "tensorwise" if recipe.scaling == "tensorwise" else "rowwise"
        x2 = x.reshape(-1, x.shape[-1])
        return _fp8_mm(x2, w, mode, x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        r = ctx.recipe
        mode = "tensorwise" if r.scaling == "tensorwise" else "rowwise"
        g2, x2 = gy.reshape(-1, gy.shape[-1]), x.reshape(-1, x.shape[-1])
        gx = _fp8_mm(g2, w.t(), mode, gy.dtype, grad=True).reshape(x.shape) if ctx.needs_input_grad[0] else None
        gw = None
        if ctx.needs_input_grad[1]:
            if r.scaling == "rowwise_with_gw_hp":
                gw = (g2.t().float() @ x2.float()).to(w.dtype)
            else:
                gw = _fp8_mm(g2.t(), x2.t(), mode, torch.float32, grad=True).to(w.dtype)
        return gx, gw, None


# ---- MXFP8 -----------------------------------------------------------------------------------
def quantize_mxfp8(x: torch.Tensor, axis: int = -1):
    """Block-scale ``x`` along ``axis`` in groups of 32: returns (e4m3 data, uint8 E8M0 exponents with
    bias 127, same shape as ``x`` with ``axis`` divided by 32). RCEIL: the exponent is
    ``ceil(log2(amax / 448))`` so that no element saturates."""
    x = x.movedim(axis, -1)
    assert x.shape[-1] % MX_BLOCK == 0, f"the scaled dimension ({x.shape[-1]}) must be a multiple of {MX_BLOCK}"
    blocks = x.float().reshape(*x.shape[:-1], x.shape[-1] // MX_BLOCK, MX_BLOCK)
    amax = blocks.abs().amax(-1, keepdim=True)
    e = torch.ceil(torch.log2(amax.clamp_min(2.0**-127 * E4M3_MAX) / E4M3_MAX)).clamp(-127, 127)
    q = (blocks * torch.exp2(-e)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    q = q.reshape(x.shape).movedim(-1, axis)
    scales = (e.squeeze(-1) + 127).to(torch.uint8).movedim(-1, axis)
    return q, scales


def dequantize_mxfp8(q: torch.Tensor, scales: torch.Tensor, axis: int = -1, dtype=torch.float32):
    q = q.movedim(axis, -1)
    s = torch.exp2(scales.movedim(axis, -1).float() - 127)
    out = q.float().reshape(*q.shape[:-1], q.shape[-1] // MX_BLOCK, MX_BLOCK) * s.unsqueeze(-1)
    return out.reshape(q.shape).movedim(-1, axis).to(dtype)


def _mx_mm(a: torch.Tensor, b_t: torch.Tensor, out_dtype):
    """``a [M,K] @ b_t [N,K]^T``, both block-scaled along K (K padded with zeros to a multiple of 32)."""
    K = a.shape[-1]
    pad = -K % MX_BLOCK
    if pad:
        a = torch.nn.functional.pad(a, (0, pad))
        b_t = torch.nn.functional.pad(b_t, (0, pad))
    from . import native

    qa_sa = qb_sb = None
    if a.is_cuda and native.has("tt_mxfp8_quant_rows"):
        from .cuda_ops import quantize_mxfp8_operand

        qa_sa, qb_sb = quantize_mxfp8_operand(a), quantize_mxfp8_operand(b_t)
    qa, sa = qa_sa if qa_sa is not None else quantize_mxfp8(a.contiguous())
    qb, sb = qb_sb if qb_sb is not None else quantize_mxfp8(b_t.contiguous())

    if a.is_cuda and native.has("tt_gemm_mxfp8"):
        from .cuda_ops import gemm_mxfp8

        return gemm_mxfp8(qa, qb, sa, sb, out_dtype)
    return (dequantize_mxfp8(qa, sa) @ dequantize_mxfp8(qb, sb).t()).to(out_dtype)


class _MxLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return _mx_mm(x.reshape(-1, x.shape[-1]), w, x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        g2, x2 = gy.reshape(-1, gy.shape[-1]), x.reshape(-1, x.shape[-1])
        gx = _mx_mm(g2, w.t(), gy.dtype).reshape(x.shape) if ctx.needs_input_grad[0] else None
        gw = _mx_mm(g2.t(), x2.t(), torch.float32).to(w.dtype) if ctx.needs_input_grad[1] else None
        return gx, gw


def quant_linear(x: torch.Tensor, w: torch.Tensor, bias, recipe: QuantRecipe):
    w = w.to_local() if hasattr(w, "to_local") else w
    y = None
    if recipe.kind == "mxfp8" and x.is_cuda and not recipe.emulate:
        from .cuda_ops import mx_linear

        y = mx_linear(x, w)            # one dispatcher-visible op per GEMM, gradient written into the FSDP slot
    if y is None:
        y = _MxLinear.apply(x, w) if recipe.kind == "mxfp8" else _Fp8Linear.apply(x, w, recipe)
    return y if bias is None else y + bias


def quant_grouped_linear(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, recipe: QuantRecipe):
    """Per-expert ``x_e @ w[e]^T`` over row groups of sizes ``counts`` with quantised GEMMs; rows past
    ``sum(counts)`` (alignment padding at the end) produce zeros. MXFP8 on CUDA with groups aligned to 128 rows runs as
    one grouped launch per GEMM with the boundaries on the device; other cases go expert by expert (one host read of
    the counts)."""
    w = w.to_local() if hasattr(w, "to_local") else w
    if recipe.kind == "mxfp8" and x.is_cuda and not recipe.emulate:
        from .cuda_ops import mx_grouped_linear

        y = mx_grouped_linear(x, w, counts)
        if y is not None:
            return y
    sizes = counts.tolist()
    outs, start = [], 0
    for e, n in enumerate(sizes):
        xe = x[start : start + n]
        if recipe.kind == "mxfp8":
            outs.append(_MxLinear.apply(xe, w[e]))
        else:
            outs.append(_Fp8Linear.apply(xe, w[e], recipe))
        start += n
    if start < x.shape[0]:
        outs.append(x.new_zeros(x.shape[0] - start, w.shape[1]))
    return torch.cat(outs, 0)
