"""Random-weights mode: write a model folder from a configuration and a seed.

``write_random_model(raw_config, out_dir, seed)`` builds the architecture named by the
configuration (without touching a GPU), asks it which tensors it needs, draws each one
from a generator keyed by ``(seed, tensor name)`` and writes ``config.json`` and
``model.safetensors``.  Matrices and embeddings are N(0, ``std``); norm gains are
``1 + N(0, gain_std)``.  Values are drawn in fp32 and stored in ``store_dtype``
(bfloat16 by default, so that a bfloat16 engine, a float32 engine and a plain fp32
implementation all see exactly the same numbers).

The reference has no such mode (its tests overwrite ``nn.Module`` defaults by hand,
``tests/unit/models/llama/test_llama_rope_scaling.py:83-92``).
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Mapping

import torch

from ..config.registry import load_config
from ..parts.model import DecoderModel
from .safetensors_io import write_safetensors


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(seed: int, name: str, shape, role: str, *, std: float, gain_std: float,
                  device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(tensor_seed(seed, name))
    t = torch.randn(tuple(shape), generator=gen, dtype=torch.float32, device=device)
    if role == "gain":
        return 1.0 + gain_std * t
    return std * t


def random_state_dict(raw_config: Mapping[str, Any], seed: int, *, std: float = 0.02,
                      gain_std: float = 0.1, std_overrides: Mapping[str, float] | None = None,
                      store_dtype: torch.dtype = torch.bfloat16, device="cpu") -> dict[str, torch.Tensor]:
    arch, cfg = load_config(raw_config)
    model = DecoderModel(arch.assemble(cfg))
    out: dict[str, torch.Tensor] = {}
    for e in model.expected_tensors():
        s = std
        for key, value in (std_overrides or {}).items():
            if key in e.name:
                s = value
        t = random_tensor(seed, e.name, e.decl.shape, e.decl.role, std=s, gain_std=gain_std, device=device)
        out[e.name] = t.to(store_dtype)
    return out


def write_random_model(raw_config: Mapping[str, Any], out_dir: str | os.PathLike, seed: int, *,
                       std: float = 0.02, gain_std: float = 0.1,
                       std_overrides: Mapping[str, float] | None = None,
                       store_dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` into ``out_dir``; return the folder."""
    out_dir = os.fspath(out_dir)
    os.makedirs(out_dir, exist_ok=True)
    state = random_state_dict(raw_config, seed, std=std, gain_std=gain_std,
                              std_overrides=std_overrides, store_dtype=store_dtype)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(raw_config), f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), state,
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
