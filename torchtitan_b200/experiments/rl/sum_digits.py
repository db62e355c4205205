"""The toy verifiable task of the RL example: add up all digits of a short list of two-digit numbers.
Behaviour follows torchtitan/experiments/rl/unified/sum_digits.py:16-106: answers are read from an
``[ANSWER] <n>`` tag, else from "answer is/answer:" phrasing, else the last number in the text;
reward +1 / -1 for right / wrong plus 0.2 when the completion is correct, has exactly one tag and ends with it."""

from __future__ import annotations

import random
import re

import torch

_TAG = re.compile(r"\[ANSWER\]\s*(-?\d+)")
_PHRASES = (
    re.compile(r"(?:the answer is|answer is|answer:)\s*(-?\d+)", re.IGNORECASE),
    re.compile(r"=\s*(-?\d+)\.?\s*(?:The answer|$)", re.IGNORECASE),
)
_NUMBER = re.compile(r"-?\d+")

SYSTEM_PROMPT = (
    "You are a careful assistant. Work through the problem one step at a time.\n"
    "Finish with the final result written as [ANSWER] <number> and write nothing after it.\n\n"
    "Example:\n"
    "User: What is the total digit sum of [12, 345, 67]?\n"
    "Assistant: Split the numbers into digits: 1, 2, 3, 4, 5, 6, 7.\n"
    "Add them: 1 + 2 + 3 + 4 + 5 + 6 + 7 = 28\n"
    "[ANSWER] 28"
)


def extract_answer(text: str) -> int | None:
    m = _TAG.findall(text)
    if m:
        return int(m[-1])
    for pat in _PHRASES:
        m = pat.findall(text)
        if m:
            return int(m[-1])
    m = _NUMBER.findall(text)
    return int(m[-1]) if m else None


class SumDigitsTask:
    """Questions over 2-4 integers in [10, 99]; deterministic for a given seed."""

    def __init__(self, seed: int = 42):
        self.seed = seed
        self._rng = random.Random(seed)

    def create_question(self) -> tuple[str, str]:
        numbers = [self._rng.randint(10, 99) for _ in range(self._rng.randint(2, 4))]
        answer = sum(int(d) for n in numbers for d in str(n))
        return f"What is the total digit sum of {numbers}?", str(answer)

    def get_system_prompt(self) -> str:
        return SYSTEM_PROMPT

    def reward_function(self, completions: list[str], expected_answer: str = "") -> torch.Tensor:
        expected = int(expected_answer) if expected_answer else 0
        out = []
        for c in completions:
            ok = extract_answer(c) == expected
            r = 1.0 if ok else -1.0
            if ok and len(re.findall(r"\[ANSWER\]", c)) == 1 and re.search(r"\[ANSWER\]\s*-?\d+\s*$", c):
                r += 0.2
            out.append(r)
        return torch.tensor(out, dtype=torch.float32)
