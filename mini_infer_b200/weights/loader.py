"""Binding checkpoint tensors to a model's parts by name.

The model says which tensors it expects (full name, shape); the checkpoint says which it
has.  All disagreements are collected and reported in one ``WeightLoadError`` before
anything is copied to the device: names the model needs and the checkpoint lacks
(missing), names the checkpoint has and nothing reads (unexpected), and shape
mismatches.  The reference reports the same three classes
(``distributed/loader.py:109-212``, ``models/llama/llama.py:203-207``).

Dtype policy (what "kept as stored" means on the device):

* engine dtype bfloat16: 16-bit floats become bfloat16, a tensor stored in 32-bit stays
  32-bit (parts that feed it to a matrix product convert their own copy), integer tables
  become int32;
* engine dtype float32: every float becomes float32 (exact for bfloat16 sources).
"""

from __future__ import annotations

import os

import torch

from .safetensors_io import Checkpoint

_INT_DTYPES = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool)


class WeightLoadError(ValueError):
    def __init__(self, message: str, missing=(), unexpected=(), mismatched=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.mismatched = list(mismatched)


def to_engine_dtype(t: torch.Tensor, engine_dtype: torch.dtype) -> torch.Tensor:
    if t.dtype in _INT_DTYPES:
        return t.to(torch.int32)
    if engine_dtype == torch.float32:
        return t.to(torch.float32)
    if t.dtype in (torch.float32, torch.float64):
        return t.to(torch.float32)
    return t.to(torch.bfloat16)


def check_names(model, names_and_shapes: dict[str, tuple[int, ...]], where: str = "checkpoint") -> None:
    """Raise one ``WeightLoadError`` listing everything that does not fit ``model``."""
    expected = {e.name: e.decl.shape for e in model.expected_tensors()}
    ignorable = model.ignorable_tensors()
    missing = sorted(n for n in expected if n not in names_and_shapes)
    unexpected = sorted(n for n in names_and_shapes if n not in expected and n not in ignorable)
    mismatched = sorted(
        (n, tuple(expected[n]), tuple(names_and_shapes[n]))
        for n in expected
        if n in names_and_shapes and tuple(names_and_shapes[n]) != tuple(expected[n])
    )
    if missing or unexpected or mismatched:
        lines = [f"weights in {where} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): {missing}")
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): {unexpected}")
        if mismatched:
            lines.append(
                f"  wrong shape ({len(mismatched)}): "
                + ", ".join(f"{n}: expected {e}, found {g}" for n, e, g in mismatched)
            )
        raise WeightLoadError("\n".join(lines), missing, unexpected, mismatched)


class TensorSource:
    """Tensors by full checkpoint name, fetched when asked for and not kept: ``model.bind`` takes
    one part's tensors at a time, so a part's own copies (a merged projection, say) are built
    while only that part's checkpoint tensors are on the device, and peak memory is the model
    plus one part, not twice the model.  (The reference loads shard by shard for the same
    reason, ``models/loader.py:188-215``.)"""

    def __init__(self, fetch) -> None:
        self._fetch = fetch

    def __getitem__(self, name: str) -> torch.Tensor:
        return self._fetch(name)


def load_weights(model, model_dir: str | os.PathLike, dtype: torch.dtype, device) -> None:
    """Read ``model_dir``'s safetensors into ``model`` (a ``DecoderModel``), part by part."""
    device = torch.device(device)
    with Checkpoint(os.fspath(model_dir)) as ckpt:
        check_names(model, {n: ckpt.shape(n) for n in ckpt.names()}, where=os.fspath(model_dir))
        model.bind(TensorSource(lambda name: to_engine_dtype(ckpt.read(name), dtype).to(device)), dtype, device)


def bind_state_dict(model, state: dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
    """Bind tensors already in memory (same checks and dtype policy as ``load_weights``)."""
    device = torch.device(device)
    check_names(model, {n: tuple(t.shape) for n, t in state.items()}, where="the given tensors")
    model.bind(TensorSource(lambda name: to_engine_dtype(state[name], dtype).to(device)), dtype, device)
