"""Sampling options of a request.

Names, defaults and checks are the reference's (``engine/sampler.py:7-21``):
``temperature`` 0 means greedy, ``top_k`` 0 and ``top_p`` 1.0 switch the filters off.
``seed`` is this engine's addition: the reference draws from torch's global generator,
here every request has a seed of its own and token ``n`` of a request is drawn from
``(seed, n)`` alone, so results do not depend on what else is in the batch.
"""

from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int | None = None

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError(f"top_p must be in [0, 1], got {self.top_p}")
        if self.seed is not None and not 0 <= self.seed < 2 ** 64:
            raise ValueError(f"seed must fit 64 bits, got {self.seed}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
