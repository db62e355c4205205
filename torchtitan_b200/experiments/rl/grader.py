"""Scores episodes with a reward function ``(completions, expected_answer) -> tensor`` (one call per
episode, as torchtitan/experiments/rl/unified/actors/grader.py:17-65). Runs on the host."""

from __future__ import annotations

from typing import Callable

import torch

from torchtitan_b200.tools.logging import logger

from .types import Episode


class Grader:
    def __init__(self, reward_fn: Callable):
        self.reward_fn = reward_fn

    def score(self, episodes: list[Episode]) -> list[Episode]:
        for ep in episodes:
            ep.reward = float(self.reward_fn([ep.text], ep.expected_answer)[0])
        if episodes:
            r = torch.tensor([ep.reward for ep in episodes])
            logger.debug(f"Grader: reward_mean={r.mean().item():.4f} reward_std={r.std().item() if len(r) > 1 else 0.0:.4f}")
        return episodes


def group_mean_advantages(episodes: list[Episode], normalize_std: bool = False) -> list[Episode]:
    """GRPO advantages: reward minus the mean reward of the episode's group (optionally divided by the
    group's standard deviation, the original GRPO form)."""
    groups: dict[str, list[int]] = {}
    for i, ep in enumerate(episodes):
        groups.setdefault(ep.group_id, []).append(i)
    for idx in groups.values():
        r = torch.tensor([float(episodes[i].reward) for i in idx])
        mean = r.mean().item()
        std = r.std().item() if (normalize_std and len(idx) > 1) else 1.0
        for i in idx:
            episodes[i].advantage = (episodes[i].reward - mean) / (std + 1e-6 if normalize_std else 1.0)
    return episodes
