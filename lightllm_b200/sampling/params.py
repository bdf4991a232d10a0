"""Per-request sampling parameters, after the reference's ``SamplingParams``
(include/lightllm/ops/sampling.h:45-78): same names, meanings and defaults."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    """``temperature`` below 1e-5 is greedy (src/ops/sampling.cpp:36); 1.0 leaves the logits as
    they are.  ``top_k`` 0 = off, else logits below the k-th largest are dropped.  ``top_p`` 1.0 =
    off, else the most probable tokens whose mass reaches ``top_p`` stay.  ``min_p`` 0.0 = off,
    else tokens below ``min_p`` times the largest probability are dropped.  ``seed`` starts the
    request's own random stream (the reference's engine re-seeds a generator with 42 at every
    step, src/engine/engine_server.cpp:2051, which makes its seed a dead letter)."""

    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 42

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-5
