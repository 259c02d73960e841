"""Batched next-token choice on the device (the kernel is ``csrc/sampling.cu``).

``DeviceSampler.sample(logits, requests)`` takes fp32 logits ``[B, V]`` and, per row, the
request's ``SamplingParams``, its seed and the index of the token being drawn, and returns
the chosen ids as an int32 device tensor without synchronising.  The reference's batched
path is ``engine/sampler.py:49-90`` (greedy rows take the argmax, sampled rows divide by
the temperature, filter with top-k and top-p, then draw).
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams


def default_seed(request_number: int) -> int:
    """Seed of a request that gave none: a fixed function of its arrival number."""
    return (0x9E3779B97F4A7C15 * (request_number + 1)) & 0xFFFF_FFFF_FFFF_FFFF


class DeviceSampler:
    def __init__(self, device) -> None:
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               draw_index: Sequence[int]) -> torch.Tensor:
        B = logits.shape[0]
        if not (len(params) == len(seeds) == len(draw_index) == B):
            raise ValueError("one SamplingParams, seed and draw index per logits row")
        out = torch.empty(B, dtype=torch.int32, device=self.device)
        if all(p.greedy for p in params):
            return ops.sample(logits, out)
        V = logits.shape[1]
        host = np.empty((6, B), dtype=np.uint32)
        host[0] = np.array([p.temperature for p in params], dtype=np.float32).view(np.uint32)
        host[1] = np.array([p.top_k if 0 < p.top_k < V else 0 for p in params], dtype=np.uint32)
        host[2] = np.array([p.top_p for p in params], dtype=np.float32).view(np.uint32)
        host[3] = np.array([s & 0xFFFFFFFF for s in seeds], dtype=np.uint32)
        host[4] = np.array([(s >> 32) & 0xFFFFFFFF for s in seeds], dtype=np.uint32)
        host[5] = np.array([d & 0xFFFFFFFF for d in draw_index], dtype=np.uint32)
        staged = torch.from_numpy(host.view(np.int32)).pin_memory().to(self.device, non_blocking=True)
        return ops.sample(
            logits, out,
            temperature=staged[0].view(torch.float32), top_k=staged[1], top_p=staged[2].view(torch.float32),
            seed_lo=staged[3], seed_hi=staged[4], draw_index=staged[5],
        )
