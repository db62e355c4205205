"""Data passed between the RL roles (fields as in torchtitan/experiments/rl/unified/types.py:13-45)."""

from dataclasses import dataclass, field


@dataclass
class Episode:
    """One prompt + completion. The generator fills the token fields, the grader ``reward``, the
    controller ``advantage`` (GRPO: reward minus the mean reward of the episodes sharing ``group_id``)."""

    policy_version: int
    prompt_token_ids: list[int]
    text: str
    token_ids: list[int]
    token_log_probs: list[float]
    expected_answer: str = ""
    reward: float = 0.0
    group_id: str = ""
    advantage: float = 0.0
    finished: bool = field(default=True)
    """False when generation stopped at ``max_tokens`` instead of an end-of-sequence token."""
