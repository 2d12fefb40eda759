"""Sampling parameters of a request."""
from __future__ import annotations

from dataclasses import dataclass

GREEDY_BELOW = 1e-5  # temperature at or below this is greedy (llm-core/src/sampler.rs:40)


@dataclass(frozen=True)
class SamplingParams:
    """Names, meanings and defaults of llm-core/src/types.rs:178-196 (``SampleParams``):
    temperature 1.0 (<= 1e-5: greedy), top_p 1.0 (off), top_k 0 (off), repetition_penalty
    1.0 (off), max_new_tokens 512. Added here: ``seed`` of the Philox draw (the reference
    draws from an unseeded generator) and ``ignore_eos`` for benchmarks."""
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    max_new_tokens: int = 512
    seed: int = 0
    ignore_eos: bool = False

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")

    @property
    def greedy(self) -> bool:
        return self.temperature <= GREEDY_BELOW

    @property
    def plain(self) -> bool:
        """Greedy with nothing that changes the logits first."""
        return self.greedy and self.repetition_penalty == 1.0
