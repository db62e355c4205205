"""Token sampling without a KV cache: the whole sequence is re-run for every new token (simple, and exactly the
training forward). ``temperature == 0`` is greedy; ``top_k`` keeps the k most likely tokens.
Parity: scripts/generate/_generation.py:10-78. For fast generation use ``experiments.rl.engine.GenerationEngine``."""

from __future__ import annotations

import torch


def multinomial_sample_one(probs: torch.Tensor, rng: torch.Generator | None = None) -> torch.Tensor:
    q = torch.empty_like(probs).exponential_(1, generator=rng)
    return torch.argmax(probs / q, dim=-1, keepdim=True).to(dtype=torch.long)


def logits_to_probs(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None) -> torch.Tensor:
    logits = logits / max(temperature, 1e-5)
    if top_k is not None:
        v, _ = torch.topk(logits, k=min(top_k, logits.size(-1)))
        logits = torch.where(logits < v.select(dim=-1, index=-1).unsqueeze(-1), -float("Inf"), logits)
    return torch.softmax(logits, dim=-1)


def generate_next_token(model, x: torch.Tensor, *, temperature: float = 1.0, top_k: int | None = None,
                        rng: torch.Generator | None = None) -> torch.Tensor:
    logits = model(x)
    if temperature == 0:
        return logits[:, -1, :].argmax(dim=-1, keepdim=True)
    return multinomial_sample_one(logits_to_probs(logits[:, -1, :].float(), temperature, top_k), rng)


@torch.no_grad()
def generate(model, input_ids: torch.Tensor, *, max_new_tokens: int, temperature: float = 1.0, top_k: int | None = None,
             seed: int | None = None) -> torch.Tensor:
    if input_ids.ndim == 1:
        input_ids = input_ids.unsqueeze(0)
    rng = None
    if seed is not None:
        rng = torch.Generator(input_ids.device).manual_seed(seed)
    out = input_ids.clone()
    for _ in range(max_new_tokens):
        nxt = generate_next_token(model, out, temperature=temperature, top_k=top_k, rng=rng)
        out = torch.cat((out, nxt), dim=1)
    return out
