"""Per-request sampling options, with the reference's names, defaults and meanings.

``temperature`` (≥ 0, default 1.0; 0 = greedy), ``top_k`` (≥ 0, default 0 = off), ``top_p`` (0 < p ≤ 1,
default 1.0 = off) are the reference's ``SampleParams`` (csrc/scheduler/sample_params.h:7-12) as the request
carries them (csrc/engine/protocol.h:39-49, which also gives ``max_output_tokens`` = 1024 and ``ignore_eos`` =
false).  ``seed`` is added: the reference seeds from the OS and cannot repeat a run
(csrc/executor/sampler.cpp:12).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    max_tokens: int = 1024
    ignore_eos: bool = False
    seed: Optional[int] = None

    def __post_init__(self) -> None:
        if not (self.temperature >= 0.0):
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if isinstance(self.top_k, bool) or not isinstance(self.top_k, int) or self.top_k < 0:
            raise ValueError(f"top_k must be an integer >= 0, got {self.top_k!r}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if isinstance(self.max_tokens, bool) or not isinstance(self.max_tokens, int) or self.max_tokens <= 0:
            raise ValueError(f"max_tokens must be a positive integer, got {self.max_tokens!r}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1
