"""Sampling options, with the reference's names, defaults and meanings
(sleuth/forge/infer/sampling.py:25-33)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingConfig:
    temperature: float = 0.8        # <= 0: greedy (argmax, first index on ties)
    top_k: int = 0                  # 0 = off
    top_p: float = 1.0              # 1.0 = off
    min_p: float = 0.0              # 0.0 = off
    repetition_penalty: float = 1.0  # 1.0 = off; > 1 makes recently used tokens less likely
    repeat_last_n: int = 64         # the penalty looks at this many recent tokens; 0 = the whole context
    no_repeat_ngram: int = 0        # 0 = off; n = never repeat a phrase of n tokens

    def __post_init__(self):
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must lie in (0, 1], got {self.top_p}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must lie in [0, 1], got {self.min_p}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be positive, got {self.repetition_penalty}")
        if self.repeat_last_n < 0 or self.no_repeat_ngram < 0:
            raise ValueError("repeat_last_n and no_repeat_ngram must be >= 0")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0

    @property
    def needs_context(self) -> bool:
        return self.repetition_penalty != 1.0 or self.no_repeat_ngram > 0
