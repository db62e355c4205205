"""Text generation without a KV cache for the checkpoint-testing script: the whole sequence goes through the training
forward for every new token (slow on purpose: it exercises exactly the code that trained the weights). Sampling is this
framework's generator-side sampler (``ops.serving.sample_top_p``: inverse-CDF draws from explicit uniforms, the same
routine the RL engine's decode loop uses), with an optional top-k filter in front. For fast generation use
``experiments.rl.engine.GenerationEngine``.

Covers what torchtitan's scripts/generate/_generation.py offers (greedy at temperature 0, temperature, top-k, seed) and
adds nucleus (top-p) sampling.
"""

from __future__ import annotations

import torch

from torchtitan_b200.ops import serving


def top_k_filter(logits: torch.Tensor, k: int | None) -> torch.Tensor:
    """Logits with everything below the k-th largest value of each row set to -inf (unchanged when ``k`` is None)."""
    if k is None or k >= logits.shape[-1]:
        return logits
    kth = torch.topk(logits, k, dim=-1).values[..., -1:]
    return logits.masked_fill(logits < kth, float("-inf"))


class TokenSampler:
    """Draws one token per row from last-position logits. The randomness is one uniform number per row taken from a
    seeded generator, so a seed reproduces a sample on any device."""

    def __init__(self, temperature: float = 1.0, top_k: int | None = None, top_p: float = 1.0, seed: int | None = None,
                 device: torch.device | str = "cpu"):
        self.temperature, self.top_k, self.top_p = float(temperature), top_k, float(top_p)
        self.rng = torch.Generator(device="cpu")
        if seed is not None:
            self.rng.manual_seed(seed)
        self.device = device

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        rows = logits.float()
        if self.temperature > 0:
            rows = top_k_filter(rows, self.top_k)
        u = torch.rand(rows.shape[0], generator=self.rng).to(rows.device)
        tokens, _ = serving.sample_top_p(rows.contiguous(), self.temperature, self.top_p, u)
        return tokens.view(-1, 1).to(torch.long)


@torch.no_grad()
def generate(model, input_ids: torch.Tensor, *, max_new_tokens: int, temperature: float = 1.0, top_k: int | None = None,
             top_p: float = 1.0, seed: int | None = None) -> torch.Tensor:
    """``input_ids`` [B, S] (or [S]) -> [B, S + max_new_tokens]."""
    ids = input_ids.unsqueeze(0) if input_ids.ndim == 1 else input_ids
    sampler = TokenSampler(temperature, top_k, top_p, seed, ids.device)
    for _ in range(max_new_tokens):
        ids = torch.cat((ids, sampler(model(ids)[:, -1, :])), dim=1)
    return ids
