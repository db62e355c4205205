"""Plain PyTorch definitions of every hot op.

These are the semantics of the framework: the CPU path (tests, gloo runs) executes them
directly, and every CUDA kernel in ``csrc/`` is tested against them in fp32.
Shapes: activations are ``[B, S, H, Dh]`` (sequence before heads) everywhere.
"""

from __future__ import annotations

import functools
import math

import torch
import torch.nn.functional as F


def linear(x, weight, bias=None):
    return F.linear(x, weight, bias)


def rms_norm(x, weight, eps: float):
    return F.rms_norm(x, (x.shape[-1],), weight, eps)


def rms_norm_fp32(x, weight, eps: float):
    """fp32-math definition the CUDA kernel implements (input/output in x.dtype)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def swiglu(gate, up):
    return F.silu(gate) * up


def _gather_table(table, seqlen: int, positions):
    """table [maxS, Dh/2, 2] (cos, sin) -> [B or 1, S, 1, Dh/2, 2]."""
    if positions is None:
        t = table[:seqlen].unsqueeze(0)
    else:
        assert positions.shape[-1] == seqlen
        t = table[positions]  # [B or 1, S, Dh/2, 2]
    return t.unsqueeze(2)


def rope(x, table, positions=None, layout: str = "interleaved"):
    """Rotate pairs of ``x`` [B,S,H,Dh] by the angles in ``table`` [maxS, Dh/2, 2].

    ``interleaved``: pair i = (x[2i], x[2i+1]) (Llama "complex" form);
    ``half``: pair i = (x[i], x[i + Dh/2]) (Qwen3/GPT-OSS "cos_sin" form).
    Math is fp32, result is cast back to ``x.dtype``.
    """
    B, S, H, D = x.shape
    t = _gather_table(table, S, positions).to(x.device)
    cos, sin = t[..., 0], t[..., 1]  # [b,S,1,D/2]
    xf = x.float()
    if layout == "interleaved":
        xr = xf.reshape(B, S, H, D // 2, 2)
        a, b = xr[..., 0], xr[..., 1]
        out = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(3)
    elif layout == "half":
        a, b = xf[..., : D // 2], xf[..., D // 2 :]
        out = torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)
    else:
        raise ValueError(f"unknown rope layout {layout}")
    return out.to(x.dtype)


def attention(q, k, v, *, causal: bool = True, scale: float | None = None,
              window: int | None = None, doc_ids=None, sinks=None, return_lse: bool = False):
    """Softmax attention on ``[B,S,H,Dh]`` tensors with grouped KV heads.

    ``window``: sliding window size (a query sees keys in (i-window, i]).
    ``doc_ids``: int tensor [B,Sk], one id per key; tokens attend only inside their own document. With fewer queries
    than keys the queries are the LAST ``Sq`` positions (the same bottom-right alignment as the causal mask).
    ``sinks``: per-head learned logit [H] joining the softmax denominator only.
    """
    B, S, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    # SDPA's is_causal mask is top-left aligned; with Sq != Sk we need the bottom-right alignment
    plain = window is None and doc_ids is None and sinks is None and not return_lse and (not causal or S == Sk)
    if plain:
        def sdpa():
            return F.scaled_dot_product_attention(
                q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                is_causal=causal, scale=scale, enable_gqa=H != Hkv,
            )

        if q.is_cuda and torch.are_deterministic_algorithms_enabled():
            # the fused library backends add dQ with atomics in backward; the math backend is reproducible bit for bit
            from torch.nn.attention import SDPBackend, sdpa_kernel

            with sdpa_kernel([SDPBackend.MATH]):
                out = sdpa()
        else:
            out = sdpa()
        return out.transpose(1, 2)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    # the score matrix is materialised: bound it by walking the queries in chunks (recomputed in backward)
    chunk = S
    while B * H * chunk * Sk * 4 > (1 << 30) and chunk > 128:
        chunk = (chunk + 1) // 2
    outs, lses = [], []
    for q0 in range(0, S, chunk):
        q1 = min(S, q0 + chunk)
        args = (q[:, q0:q1], k, v, sinks, doc_ids[:, Sk - S + q0 : Sk - S + q1] if doc_ids is not None else None, doc_ids)
        fn = functools.partial(_masked_attention_rows, q0=q0 + (Sk - S), causal=causal, scale=scale, window=window)
        if chunk < S and torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, sinks)):
            from torch.utils.checkpoint import checkpoint

            o, l = checkpoint(fn, *args, use_reentrant=False)
        else:
            o, l = fn(*args)
        outs.append(o)
        lses.append(l)
    out = outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)
    if return_lse:
        return out, (lses[0] if len(lses) == 1 else torch.cat(lses, dim=2))  # lse [B,H,S]
    return out


def _masked_attention_rows(q, k, v, sinks, doc_q, doc_k, *, q0: int, causal: bool, scale: float, window):
    """Rows ``q0 ... q0 + q.shape[1]`` (key-aligned positions) of masked attention; returns (out, lse)."""
    B, S, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    qf = q.float().transpose(1, 2)  # B,H,S,D
    kf = k.float().transpose(1, 2).repeat_interleave(g, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale  # B,H,S,Sk
    qi = torch.arange(S, device=q.device).view(S, 1) + q0
    ki = torch.arange(Sk, device=q.device).view(1, Sk)
    mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device)
    if causal:
        mask &= ki <= qi
    if window is not None:
        mask &= ki > qi - window
    mask = mask.view(1, 1, S, Sk)
    if doc_q is not None:
        mask = mask & (doc_q.view(B, 1, S, 1) == doc_k.view(B, 1, 1, Sk))
    s = s.masked_fill(~mask, float("-inf"))
    if sinks is not None:
        sink = sinks.float().view(1, H, 1, 1).expand(B, H, S, 1)
        lse = torch.logsumexp(torch.cat((s, sink), dim=-1), dim=-1)
    else:
        lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    return torch.matmul(p, vf).transpose(1, 2).to(q.dtype), lse


def cross_entropy_sum(logits, labels, ignore_index: int = -100):
    """Sum over tokens of CE in fp32; rows whose label == ignore_index add 0."""
    return F.cross_entropy(
        logits.flatten(0, -2).float(), labels.flatten(), reduction="sum", ignore_index=ignore_index
    )


def token_logprobs(logits, labels):
    """log softmax(logits)[label] per token, fp32."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    return lp.gather(-1, labels.unsqueeze(-1)).squeeze(-1)


# --------------------------------------------------------------------------- MoE
def grouped_linear(x, w, counts):
    """Per-group ``x_g @ w[g].T``: ``x`` [T,K] holds the groups back to back, ``w`` [E,N,K],
    ``counts`` [E] rows per group. Rows past ``sum(counts)`` (alignment padding) give zeros."""
    out = x.new_zeros(x.shape[0], w.shape[1])
    start = 0
    for e, n in enumerate(counts.tolist()):
        n = int(n)
        if n:
            out[start : start + n] = x[start : start + n] @ w[e].transpose(-1, -2).to(x.dtype)
        start += n
    return out


def moe_route(x, gate_weight, gate_bias, expert_bias, *, top_k: int, score_func: str,
              route_norm: bool, route_scale: float, num_expert_groups=None, num_limited_groups=None,
              force_balance: bool = False):
    """Token-choice routing: fp32 gate -> scores -> (bias only for choosing) -> top-k.

    Returns (top_scores [T,k] fp32, expert index [T,k] int64, tokens per expert [E] fp32).
    """
    E = gate_weight.shape[0]
    logits = F.linear(x.float(), gate_weight.float(), None if gate_bias is None else gate_bias.float())
    if score_func == "sigmoid":
        scores = torch.sigmoid(logits)
    elif score_func == "softmax":
        scores = F.softmax(logits, dim=1)
    else:
        raise NotImplementedError(f"Unknown score function {score_func}")
    choice = scores if expert_bias is None else scores + expert_bias
    if num_expert_groups is not None:
        if num_limited_groups is None:
            raise ValueError("num_limited_groups must be set when num_expert_groups is set")
        if E % num_expert_groups != 0:
            raise ValueError(f"num_experts ({E}) must be divisible by num_expert_groups ({num_expert_groups})")
        per = E // num_expert_groups
        if per < 2:
            raise ValueError(f"experts_per_group ({per}) must be >= 2")
        grouped = choice.view(-1, num_expert_groups, per)
        gscore = grouped.topk(2, dim=-1)[0].sum(-1)
        keep = gscore.topk(num_limited_groups, dim=-1, sorted=False)[1]
        drop = torch.ones_like(gscore, dtype=torch.bool).scatter_(1, keep, False)
        choice = grouped.masked_fill(drop.unsqueeze(-1), float("-inf")).view(-1, E)
    idx = choice.topk(top_k, dim=-1, sorted=False)[1]
    if force_balance:
        T = scores.shape[0]
        idx = torch.arange(T * top_k, device=x.device, dtype=torch.int64).view(T, top_k) % E
    top = scores.gather(1, idx)
    if route_norm:
        top = top / (top.sum(-1, keepdim=True) + 1e-20)
    top = top * route_scale
    counts = torch.bincount(idx.flatten(), minlength=E).to(torch.float32)
    return top, idx, counts


def moe_sort(expert_idx, num_experts: int):
    """Stable sort of the T*k (token, slot) pairs by expert. Returns (order [T*k] int64 with
    ``order[j]`` = flat pair index placed at sorted row j, counts [E] int64)."""
    flat = expert_idx.flatten()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    return order, counts


def padded_group_layout(counts, align: int):
    """Row offsets when every group is padded up to a multiple of ``align`` (>= align rows when
    the group is empty is NOT added: empty groups take 0 rows).
    Returns (padded_counts [E], starts [E]) as int64 tensors."""
    padded = (counts + align - 1) // align * align
    starts = torch.cumsum(padded, 0) - padded
    return padded, starts
