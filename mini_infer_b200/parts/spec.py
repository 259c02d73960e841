"""Descriptions of a model as data: parts, layers, and the order layers run in.

An architecture's ``assemble(config)`` returns a :class:`ModelSpec`.  It names,
for every layer, the *kind* of each part (a key of ``parts.registry``) together
with the sizes and constants that part needs, and the prefix under which the
part's tensors live in the checkpoint.  The engine builds parts from these
descriptions; no part ever sees the configuration or knows which model it is in.

``schedule`` is the order of execution.  An entry names the layer to run (its
weights), the cache layer it uses, and whether it writes that cache.  A layer
may appear twice (shared weights, each run with a cache layer of its own), and
a layer may read a cache layer that another layer wrote
(``writes_cache=False``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part: a registered ``kind``, its parameters, and its tensor-name prefix.

    ``rename`` maps a part's local tensor name to a full checkpoint name where
    ``prefix + local`` is not the checkpoint's name.
    """

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""
    rename: Mapping[str, str] = field(default_factory=dict)

    def tensor_name(self, local: str) -> str:
        return self.rename.get(local, self.prefix + local)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer and a feed-forward, each behind a norm, in an arrangement.

    ``arrangement`` is a registered block-arrangement kind (where the norms and
    the residual additions stand).  ``position`` is the position encoding the
    mixer applies (``None``: the mixer uses none).
    """

    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    position: PartSpec | None = None
    arrangement: str = "prenorm"


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, their run order, final norm, output head."""

    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    final_norm: PartSpec
    head: PartSpec
    schedule: tuple[ScheduleEntry, ...] = ()
    max_positions: int | None = None

    def __post_init__(self) -> None:
        if not self.schedule:
            object.__setattr__(
                self,
                "schedule",
                tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(self.layers))),
            )
        n_cache = self.num_cache_layers
        writers = {e.cache for e in self.schedule if e.writes_cache}
        seen: set[int] = set()
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}, model has {len(self.layers)}")
            if not 0 <= e.cache < n_cache:
                raise ValueError(f"schedule names cache layer {e.cache} of {n_cache}")
            if e.writes_cache:
                if e.cache in seen:
                    raise ValueError(f"cache layer {e.cache} is written by two schedule entries")
                seen.add(e.cache)
            elif e.cache not in seen:
                raise ValueError(
                    f"schedule entry reads cache layer {e.cache} before any entry wrote it"
                )
        if writers != set(range(n_cache)):
            raise ValueError("every cache layer must be written by exactly one schedule entry")

    @property
    def num_cache_layers(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)
