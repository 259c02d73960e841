"""Greedy, temperature, top-k and top-p sampling."""

from .params import SamplingParams  # noqa: F401
from .sampler import DeviceSampler, default_seed  # noqa: F401
