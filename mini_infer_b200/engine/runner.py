"""``ModelRunner``: a loaded model, its cache and its step function in one object.

``ModelRunner.from_pretrained(model_dir, dtype=..., num_blocks=..., block_size=...)`` follows
the reference's constructor of the same name (``engine/model_runner.py:84-175``; the option
names ``num_blocks`` and ``block_size`` and their defaults 1024 and 16 are the reference's),
reduced to what a single-GPU engine for local model folders needs.
"""

from __future__ import annotations

import os
from typing import Any, Mapping, Sequence

import torch

from ..cache.manager import CacheManager
from ..config.registry import load_config
from ..parts.model import DecoderModel
from ..weights.loader import bind_state_dict, load_weights
from .step import StepEntry, StepResult, StepRunner

DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32,
    torch.bfloat16: torch.bfloat16, torch.float32: torch.float32,
}

DEFAULT_NUM_BLOCKS = 1024
DEFAULT_BLOCK_SIZE = 16


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"the engine runs on a CUDA device only, got {device}")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; the engine has no CPU path")
    return device


class ModelRunner:
    def __init__(self, model: DecoderModel, config: Any, *, num_blocks: int = DEFAULT_NUM_BLOCKS,
                 block_size: int = DEFAULT_BLOCK_SIZE, max_requests: int = 64,
                 cuda_graph: bool = False) -> None:
        self.model = model
        self.config = config
        self.dtype = model.dtype
        self.device = model.device
        self.cache = CacheManager(
            model.cache_needs(), page_size=block_size, num_pages=num_blocks,
            max_requests=max_requests, dtype=self.dtype, device=self.device,
            max_request_tokens=model.spec.max_positions,
        )
        self.stepper = StepRunner(model, self.cache, cuda_graph=cuda_graph)
        self.vocab_size = model.spec.vocab_size
        self.max_positions = model.spec.max_positions
        self.num_blocks = num_blocks
        self.block_size = block_size

    @classmethod
    def from_pretrained(cls, model_dir: str | os.PathLike, *, device="cuda:0", dtype="bfloat16",
                        num_blocks: int = DEFAULT_NUM_BLOCKS, block_size: int = DEFAULT_BLOCK_SIZE,
                        max_requests: int = 64, cuda_graph: bool = False) -> "ModelRunner":
        """Load ``config.json`` and the safetensors of a local model folder.  ``cuda_graph``
        replays decode-only steps as captured CUDA graphs (the reference's option of that name)."""
        device = require_cuda(device)
        tdtype = resolve_dtype(dtype)
        arch, cfg = load_config(model_dir)
        model = DecoderModel(arch.assemble(cfg))
        load_weights(model, model_dir, tdtype, device)
        return cls(model, cfg, num_blocks=num_blocks, block_size=block_size, max_requests=max_requests,
                   cuda_graph=cuda_graph)

    @classmethod
    def from_state_dict(cls, raw_config: Mapping[str, Any], state: Mapping[str, torch.Tensor], *,
                        device="cuda:0", dtype="bfloat16", num_blocks: int = DEFAULT_NUM_BLOCKS,
                        block_size: int = DEFAULT_BLOCK_SIZE, max_requests: int = 64,
                        cuda_graph: bool = False) -> "ModelRunner":
        """Build from a raw configuration mapping and tensors already in memory."""
        device = require_cuda(device)
        tdtype = resolve_dtype(dtype)
        arch, cfg = load_config(raw_config)
        model = DecoderModel(arch.assemble(cfg))
        bind_state_dict(model, dict(state), tdtype, device)
        return cls(model, cfg, num_blocks=num_blocks, block_size=block_size, max_requests=max_requests,
                   cuda_graph=cuda_graph)

    @classmethod
    def from_random(cls, raw_config: Mapping[str, Any], seed: int, *, device="cuda:0", dtype="bfloat16",
                    num_blocks: int = DEFAULT_NUM_BLOCKS, block_size: int = DEFAULT_BLOCK_SIZE,
                    max_requests: int = 64, cuda_graph: bool = False, std: float = 0.02,
                    gain_std: float = 0.1, std_overrides: Mapping[str, float] | None = None) -> "ModelRunner":
        """Build from a raw configuration mapping with the random weights of ``seed`` (the ones
        ``write_random_model`` writes), drawn on the device part by part: a model of tens of
        gigabytes needs neither a file nor host memory, and nothing exists twice."""
        from ..weights.random_init import bind_random

        device = require_cuda(device)
        tdtype = resolve_dtype(dtype)
        arch, cfg = load_config(raw_config)
        model = DecoderModel(arch.assemble(cfg))
        bind_random(model, seed, tdtype, device, std=std, gain_std=gain_std, std_overrides=std_overrides)
        return cls(model, cfg, num_blocks=num_blocks, block_size=block_size, max_requests=max_requests,
                   cuda_graph=cuda_graph)

    # -- requests -----------------------------------------------------------------------

    def add_request(self, rid) -> int:
        return self.cache.add_request(rid)

    def free_request(self, rid) -> None:
        self.cache.free_request(rid)

    # a scheduler may feed the sampler's device output to the next step (see StepRunner.step)
    device_token_feedback = True

    def step(self, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None = None) -> StepResult:
        return self.stepper.step(entries, device_tokens)

    def capture_decode_steps(self, max_batch: int) -> int:
        """Capture the decode step of every batch size up to ``max_batch`` that has no graph yet
        (a step of a new size otherwise runs kernel by kernel and is captured when it first
        occurs, some 40 ms in the middle of serving).  Uses requests of its own that hold one
        token each and gives their pages back; needs that many free pages and request slots.
        Returns the number of graphs captured; 0 when steps are not captured at all."""
        if not self.stepper.cuda_graph:
            return 0
        made = 0
        max_batch = min(max_batch, self.cache.max_requests - self.cache.num_requests)
        for b in range(1, max_batch + 1):
            slot = self.stepper._graphs.get((b,))
            if slot is not None and slot.graph is not None:
                continue
            rids = [("__capture__", i) for i in range(b)]
            for r in rids:
                self.cache.add_request(r)
            try:
                if not self.cache.can_append([(r, 1) for r in rids]):
                    break
                self.stepper.step([StepEntry(r, [0], [0]) for r in rids])   # runs kernel by kernel once, then records
                made += 1
            finally:
                for r in rids:
                    self.cache.free_request(r)
        return made

    # -- health -------------------------------------------------------------------------

    def health_word(self) -> torch.Tensor:
        """An int32 tensor of one element on the device: non-zero once a kernel has given up one
        of its bounded waits (its output, and everything computed from it, is then invalid).  A
        scheduler copies it to the host together with each step's tokens."""
        from ..csrc import ops

        return ops.status_word(self.device)

    def reset_health(self) -> None:
        """Clear the word and whatever the interrupted kernels left behind (synchronises)."""
        from ..csrc import ops

        ops.recover_from_wait_failure(self.device)
