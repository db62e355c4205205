"""Policy-gradient objectives over generated tokens.

``compute_token_log_probs`` and the ``grpo`` objective follow
torchtitan/experiments/rl/unified/actors/utils.py:11-147: per-token log-probabilities of the
completion under a model (fp32 log-softmax of the logits at the positions that predict the generated
tokens); per-sample ratio = exp(mean token log-ratio against the frozen reference), PPO clipping with
``ppo_clip_eps``, entropy bonus ``-entropy_coef * (-mean logp)``, and the k3 KL estimator
``r - 1 - log r`` averaged per sample, weighted by ``kl_coef``. ``dapo`` is the token-level variant:
importance ratios against the *generator's* log-probabilities, asymmetric clipping (``clip_low``,
``clip_high``), one mean over all tokens of the batch, no KL term.

All sequences of a step are packed into one row with document masking, so a step is one forward pass
regardless of the number of episodes; log-probabilities come from the chunked cross-entropy kernel
and the fp32 ``[tokens, vocab]`` log-softmax is never materialised.
"""

from __future__ import annotations

import torch

from torchtitan_b200 import ops
from torchtitan_b200.models.common.attention import AttentionMasks


def pack_sequences(prompt_token_ids: list[list[int]], gen_token_ids: list[list[int]], device, pad_to: int = 1):
    """Concatenate ``prompt + completion`` sequences into one row.

    Returns tokens [1, T], positions [1, T], document ids [1, T] and, per sequence, the (start, end) slice
    of the *logit* positions that predict its generated tokens."""
    toks, pos, doc, spans = [], [], [], []
    off = 0
    for i, (p, g) in enumerate(zip(prompt_token_ids, gen_token_ids)):
        n = len(p) + len(g)
        toks += list(p) + list(g)
        pos += list(range(n))
        doc += [i] * n
        spans.append((off + len(p) - 1, off + len(p) - 1 + len(g)))
        off += n
    pad = -off % pad_to
    if pad:
        toks += [0] * pad
        pos += list(range(pad))
        doc += [len(prompt_token_ids)] * pad
    t = torch.tensor(toks, dtype=torch.long, device=device).unsqueeze(0)
    return (t, torch.tensor(pos, dtype=torch.int32, device=device).unsqueeze(0),
            torch.tensor(doc, dtype=torch.int32, device=device).unsqueeze(0), spans)


def compute_token_log_probs_packed(model, prompt_token_ids, gen_token_ids, device, pad_to: int = 1) -> list[torch.Tensor]:
    """Per-token log-probabilities of every completion, one packed forward pass."""
    tokens, positions, doc, spans = pack_sequences(prompt_token_ids, gen_token_ids, device, pad_to)
    masks = AttentionMasks(doc_ids=doc)
    logits = _forward_packed(model, tokens, masks, positions)
    labels = torch.roll(tokens, -1, dims=1)
    lp = ops.token_logprobs(logits[0], labels[0])          # [T] fp32, log p(label_t | prefix)
    return [lp[s:e] for s, e in spans]


def _forward_packed(model, tokens, masks, positions):
    """Run a decoder on a packed row with per-document attention regardless of its configured backend."""
    h = model.tok_embeddings(tokens) if model.tok_embeddings is not None else tokens
    for layer in model.layers.values():
        att = layer.attention
        saved = getattr(att, "attn_backend", None)
        if saved == "sdpa":
            att.attn_backend = "flex"       # the packed row needs the document mask
        try:
            h = layer(h, model.freqs_cis, masks, positions)
        finally:
            if saved is not None:
                att.attn_backend = saved
    h = model.norm(h) if model.norm is not None else h
    return model.output(h) if model.output is not None else h


def compute_token_log_probs(model, prompt_token_ids: list[int], gen_token_ids: list[int], device) -> torch.Tensor:
    """Single-sequence form (kept for parity with the reference helper)."""
    return compute_token_log_probs_packed(model, [prompt_token_ids], [gen_token_ids], device)[0]


def compute_policy_gradient_loss(model, gen_token_ids, prompt_token_ids, advantages, ref_token_log_probs,
                                 kl_coef: float = 0.1, ppo_clip_eps: float = 0.2, entropy_coef: float = 0.01,
                                 objective: str = "grpo", gen_token_log_probs=None, clip_low: float = 0.2,
                                 clip_high: float = 0.28, pad_to: int = 1, n_seqs_total: int | None = None,
                                 n_tokens_total: int | None = None):
    """Loss of one (micro-)batch. ``n_seqs_total`` / ``n_tokens_total`` are the counts of the whole step when the
    episodes are processed in several micro-batches: every mean below divides by them, so the micro-batch losses add up
    to the loss of the full batch and gradients can simply be accumulated."""
    device = next(model.parameters()).device
    advantages = advantages.to(device)
    token_lps = compute_token_log_probs_packed(model, prompt_token_ids, gen_token_ids, device, pad_to)
    all_lps = torch.cat(token_lps)
    n_seq = float(n_seqs_total if n_seqs_total is not None else len(token_lps))
    n_tok = float(n_tokens_total if n_tokens_total is not None else max(1, all_lps.numel()))
    entropy = -all_lps.sum() / n_tok
    if objective == "dapo":
        assert gen_token_log_probs is not None, "the dapo objective needs the generator's log-probabilities"
        old = torch.cat([torch.as_tensor(o, dtype=torch.float32, device=device) for o in gen_token_log_probs])
        adv = torch.cat([advantages[i].expand(len(t)) for i, t in enumerate(token_lps)])
        ratio = torch.exp(all_lps - old)
        clipped = ratio.clamp(1 - clip_low, 1 + clip_high)
        pg_loss = -torch.min(ratio * adv, clipped * adv).sum() / n_tok
        kl_div = torch.zeros((), device=device)
        total = pg_loss - entropy_coef * entropy
    else:
        log_ratio, kls = [], []
        for pol, ref in zip(token_lps, ref_token_log_probs):
            lr = pol - ref.detach()
            log_ratio.append(lr.mean())
            kls.append((torch.exp(lr) - 1 - lr).mean())
        ratio = torch.exp(torch.stack(log_ratio))
        clipped = ratio.clamp(1 - ppo_clip_eps, 1 + ppo_clip_eps)
        pg_loss = -torch.min(ratio * advantages, clipped * advantages).sum() / n_seq
        kl_div = torch.stack(kls).sum() / n_seq
        total = pg_loss - entropy_coef * entropy + kl_coef * kl_div
    metrics = {
        "pg_loss": pg_loss.item(), "entropy": entropy.item(), "kl_div": kl_div.item(), "ratio_mean": ratio.mean().item(),
        "ratio_clipped_frac": ((ratio - clipped).abs() > 1e-6).float().mean().item(),
    }
    return total, metrics, token_lps


def verify_logprob_identity(gen_token_log_probs: list[list[float]], batch_token_log_probs: list[torch.Tensor]) -> dict:
    """Compare generator and trainer log-probabilities token by token."""
    res = {"logprob_bitwise_identical": True, "num_samples_checked": len(gen_token_log_probs), "total_tokens_checked": 0,
           "num_tokens_different": 0, "logprob_max_delta": 0.0, "avg_delta": 0.0, "logprob_diff_mean": 0.0,
           "logprob_diff_max": 0.0}
    deltas, ratios = [], []
    for g, t in zip(gen_token_log_probs, batch_token_log_probs):
        gt = torch.tensor(g, dtype=torch.float32)
        tt = t.detach().cpu().float()
        res["total_tokens_checked"] += len(g)
        if not torch.equal(gt, tt):
            res["logprob_bitwise_identical"] = False
            res["num_tokens_different"] += int((gt != tt).sum())
            deltas.append((gt - tt).abs())
        ratios.append(tt - gt)
    if deltas:
        d = torch.cat(deltas)
        res["logprob_max_delta"], res["avg_delta"] = d.max().item(), d.mean().item()
    if ratios:
        r = torch.cat(ratios)
        if r.numel():
            res["logprob_diff_mean"], res["logprob_diff_max"] = r.mean().item(), r.abs().max().item()
    return res
