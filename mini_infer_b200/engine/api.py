"""The Python entry point, in the reference's manner (``README.md:108-131``):

    runner = ModelRunner.from_pretrained(model_dir, dtype="bfloat16", num_blocks=1024, block_size=16)
    scheduler = ContinuousScheduler(runner, max_concurrent=16)
    result = scheduler.run(Request(prompt=[1, 2, 3], sampling_params=SamplingParams(), max_tokens=32))
    result.tokens, result.finish_reason

``generate_ids`` wraps those three lines for callers that have token ids and want token ids.
"""

from __future__ import annotations

from typing import Sequence

from ..sampling.params import SamplingParams
from .runner import DEFAULT_BLOCK_SIZE, DEFAULT_NUM_BLOCKS, ModelRunner
from .scheduler import ContinuousScheduler, GenerationResult, Request


def generate(runner: ModelRunner, prompts: Sequence[Sequence[int]], *, max_tokens: int = 16,
             sampling_params: SamplingParams | Sequence[SamplingParams] | None = None,
             max_concurrent: int = 16, chunk_size: int | None = None, max_tokens_per_step: int = 2048,
             decode_headroom_blocks: int = 8, eos_token_ids: Sequence[int] = ()) -> list[GenerationResult]:
    """Generate for every prompt (token ids) with continuous batching; results in order."""
    if sampling_params is None:
        sampling_params = SamplingParams()
    if isinstance(sampling_params, SamplingParams):
        sampling_params = [sampling_params] * len(prompts)
    scheduler = ContinuousScheduler(
        runner, max_concurrent=max_concurrent, chunk_size=chunk_size,
        max_tokens_per_step=max_tokens_per_step, decode_headroom_blocks=decode_headroom_blocks,
        eos_token_ids=eos_token_ids,
    )
    return scheduler.generate(
        [Request(prompt=list(p), sampling_params=sp, max_tokens=max_tokens)
         for p, sp in zip(prompts, sampling_params)]
    )


def generate_ids(model_dir: str, prompts: Sequence[Sequence[int]], *, max_tokens: int = 16,
                 dtype: str = "bfloat16", device: str = "cuda:0", temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int | None = None,
                 num_blocks: int = DEFAULT_NUM_BLOCKS, block_size: int = DEFAULT_BLOCK_SIZE) -> list[list[int]]:
    """Load ``model_dir`` and return the generated token ids of every prompt."""
    runner = ModelRunner.from_pretrained(model_dir, device=device, dtype=dtype, num_blocks=num_blocks,
                                         block_size=block_size,
                                         max_requests=max(1, min(64, len(prompts))))
    params = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed)
    return [r.tokens for r in generate(runner, prompts, max_tokens=max_tokens, sampling_params=params)]
