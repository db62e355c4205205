"""Generation-side ops: paged-KV decode attention, KV-cache writes and the token sampler.

PyTorch definitions (any device) and dispatch to the native kernels on CUDA. The cache layout is
``[num_blocks, block_size, n_kv_heads, head_dim]`` for keys and values; ``block_tables[b, i]`` is the
cache block holding tokens ``i*block_size ... (i+1)*block_size-1`` of sequence ``b``.

Reference counterpart: vLLM's paged attention and sampler as used by
torchtitan/experiments/rl/unified/models/attention.py:62-117 and actors/generator.py:251-260
(temperature, top-p, sampled-token log-probability from an fp32 log-softmax of the raw logits).
"""

from __future__ import annotations

import torch

from . import native


def kv_cache_write(k_cache, v_cache, k, v, slots):
    """Scatter new keys/values ``[T, Hkv, D]`` into flat cache slots ``slots[T]`` (= block * block_size + offset)."""
    if k.is_cuda and native.has("tt_kv_write"):
        from .cuda_ops import kv_write

        return kv_write(k_cache, v_cache, k, v, slots)
    kc, vc = k_cache.view(-1, *k_cache.shape[2:]), v_cache.view(-1, *v_cache.shape[2:])
    kc.index_copy_(0, slots.long(), k.to(kc.dtype))
    vc.index_copy_(0, slots.long(), v.to(vc.dtype))


def paged_attention_decode(q, k_cache, v_cache, block_tables, context_lens, scale: float):
    """One query token per sequence: ``q [B, H, D]`` attends to the first ``context_lens[b]`` cached tokens
    of its sequence. Returns ``[B, H, D]``. GQA: query head h reads kv head ``h // (H / Hkv)``."""
    if q.is_cuda and native.has("tt_paged_decode") and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and \
            (q.shape[1] // k_cache.shape[2]) in (1, 2, 4, 8):
        from .cuda_ops import paged_decode

        return paged_decode(q, k_cache, v_cache, block_tables, context_lens, scale)
    B, H, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    max_ctx = block_tables.shape[1] * bs
    idx = (block_tables.long().unsqueeze(-1) * bs + torch.arange(bs, device=q.device)).view(B, max_ctx)
    k = k_cache.view(-1, Hkv, D)[idx]            # [B, ctx, Hkv, D]
    v = v_cache.view(-1, Hkv, D)[idx]
    rep = H // Hkv
    k = k.repeat_interleave(rep, dim=2).float()
    v = v.repeat_interleave(rep, dim=2).float()
    s = torch.einsum("bhd,bchd->bhc", q.float(), k) * scale
    dead = torch.arange(max_ctx, device=q.device).view(1, 1, -1) >= context_lens.view(B, 1, 1)
    s = s.masked_fill(dead, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhc,bchd->bhd", p, v).to(q.dtype)


def sample_top_p(logits, temperature: float, top_p: float, uniforms):
    """Sample one token per row of ``logits [B, V]``.

    ``uniforms [B]`` in [0, 1) drives the draw by inverse CDF in vocabulary index order -- over the whole vocabulary
    when ``top_p >= 1`` (plain multinomial sampling), over the nucleus otherwise -- so a given (logits, uniform) pair
    yields the same token on every device up to rounding at CDF boundaries. The nucleus is the set of tokens at least as
    likely as the last token needed to reach a cumulative mass of ``top_p`` from the most likely down (ties at that
    probability are all kept).
    ``temperature == 0`` is greedy (lowest index on ties). Returns (tokens int64 [B], log-probabilities fp32 [B]); the log-probability is taken from the
    fp32 log-softmax of the *unscaled* logits, which is what the trainer recomputes."""
    if logits.is_cuda and native.has("tt_sample") and (top_p >= 1.0 or temperature <= 0.0 or native.has("tt_sample_top_p")):
        from .cuda_ops import sample as native_sample

        return native_sample(logits, temperature, uniforms, top_p)
    lf = logits.float()
    logp_raw = torch.log_softmax(lf, dim=-1)
    if temperature <= 0.0:
        tok = lf.argmax(-1)
        return tok, logp_raw.gather(1, tok.view(-1, 1)).squeeze(1)
    probs = torch.softmax(lf / temperature, dim=-1)
    if top_p >= 1.0:
        cdf = probs.cumsum(-1)
        target = uniforms.float().view(-1, 1) * cdf[:, -1:]
        tok = (cdf <= target).sum(-1).clamp(max=logits.shape[-1] - 1)
        return tok, logp_raw.gather(1, tok.view(-1, 1)).squeeze(1)
    keep = nucleus_mask(probs, top_p)
    cdf = (probs * keep).cumsum(-1)
    target = uniforms.float().view(-1, 1) * cdf[:, -1:]
    tok = (cdf <= target).sum(-1)
    last_kept = logits.shape[-1] - 1 - keep.flip(-1).float().argmax(-1)
    tok = torch.minimum(tok, last_kept)
    return tok, logp_raw.gather(1, tok.view(-1, 1)).squeeze(1)


def nucleus_mask(probs, top_p: float):
    """Boolean [B, V]: tokens whose probability is >= that of the last token taken when accumulating ``top_p`` of mass
    from the most likely token down (the most likely token is always in)."""
    sp, _ = probs.sort(dim=-1, descending=True)
    taken = (sp.cumsum(-1) - sp) < top_p
    cut = torch.where(taken, sp, torch.full_like(sp, float("inf"))).amin(-1, keepdim=True)
    return probs >= cut
