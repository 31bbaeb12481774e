"""SamplingParams: the reference's five options
(python/lyapunov_engine/engine/sampling.py:6-12) with the same names, meanings
and defaults, plus a seed."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 1.0   # below 1e-4: greedy
    top_p: float = 1.0         # keep the smallest set of most likely tokens whose mass reaches top_p
    top_k: int = -1            # keep the k most likely tokens; <= 0: all
    max_tokens: int = 128
    ignore_eos: bool = False
    seed: int = 0              # the draw for a token depends on (seed, index of the token) only

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-4
