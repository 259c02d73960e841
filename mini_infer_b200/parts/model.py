"""A decoder built from a :class:`~.spec.ModelSpec`.

``DecoderModel`` owns the built parts, knows the full checkpoint name of every tensor
they declared, hands loaded tensors to them, and runs one step: embedding, the schedule
of layers, final norm and output head on the wanted rows only.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import (
    Arrangement,
    KVNeed,
    LayerCache,
    ParamDecl,
    Part,
    PlanNeeds,
    StateNeed,
    StepContext,
    build_part,
    lookup,
)
from .spec import ModelSpec, PartSpec


@dataclass(frozen=True)
class ExpectedTensor:
    name: str            # full checkpoint name
    decl: ParamDecl
    part: Part
    local: str


@dataclass(frozen=True)
class CacheLayerNeed:
    """What cache layer ``index`` must hold (from the mixer of the entry that writes it)."""

    index: int
    kv: KVNeed | None
    state: StateNeed | None


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.blocks: list[Arrangement] = []
        for layer in spec.layers:
            position = build_part("position", layer.position) if layer.position else None
            block = lookup("arrangement", layer.arrangement)(
                build_part("mixer", layer.mixer),
                build_part("feed_forward", layer.feed_forward),
                build_part("norm", layer.mixer_norm),
                build_part("norm", layer.feed_forward_norm),
                position,
            )
            self.blocks.append(block)
        self.schedule = spec.schedule
        self._bound = False

    # ------------------------------------------------------------------ declarations

    def all_parts(self) -> list[Part]:
        parts: list[Part] = [self.embedding]
        for b in self.blocks:
            parts.extend(b.parts())
        parts.extend([self.final_norm, self.head])
        return parts

    def expected_tensors(self) -> list[ExpectedTensor]:
        out: list[ExpectedTensor] = []
        seen: dict[str, ExpectedTensor] = {}
        for part in self.all_parts():
            for local, decl in part.param_decls().items():
                name = part.spec.tensor_name(local)
                if name in seen:
                    if seen[name].decl.shape != decl.shape:
                        raise ValueError(
                            f"tensor {name!r} is declared twice with shapes "
                            f"{seen[name].decl.shape} and {decl.shape}"
                        )
                    continue
                e = ExpectedTensor(name, decl, part, local)
                seen[name] = e
                out.append(e)
        return out

    def ignorable_tensors(self) -> set[str]:
        """Names a checkpoint may carry although nothing reads them (a tied head's copy)."""
        head = self.head
        if getattr(head, "tied", False):
            return {head.spec.tensor_name("weight")}
        return set()

    def cache_needs(self) -> list[CacheLayerNeed]:
        needs: dict[int, CacheLayerNeed] = {}
        for e in self.schedule:
            mixer = self.blocks[e.layer].mixer
            kv, st = mixer.cache_need(), mixer.state_need()
            if e.writes_cache:
                needs[e.cache] = CacheLayerNeed(e.cache, kv, st)
        for e in self.schedule:
            if not e.writes_cache:
                mixer = self.blocks[e.layer].mixer
                kv, owner = mixer.cache_need(), needs[e.cache].kv
                if kv is None or owner is None or (kv.kv_heads, kv.head_dim) != (owner.kv_heads, owner.head_dim):
                    raise ValueError(
                        f"layer {e.layer} reads cache layer {e.cache} whose key/value shape "
                        f"{owner} does not fit its own {kv}"
                    )
        return [needs[i] for i in range(self.spec.num_cache_layers)]

    def plan_needs(self) -> PlanNeeds:
        tiles: set[int] = set()
        for b in self.blocks:
            tiles |= set(b.mixer.plan_needs().q_tile_tokens)
        return PlanNeeds(frozenset(tiles))

    def graph_safe(self) -> bool:
        """Whether a step of this model may be captured as a CUDA graph (every part says so)."""
        return all(p.graph_safe for p in self.all_parts())

    # ------------------------------------------------------------------ binding

    def bind(self, tensors, dtype: torch.dtype, device: torch.device) -> None:
        """Give every part its tensors.  ``tensors`` is anything indexed by full checkpoint
        name: a dict, or a source that fetches a tensor when it is asked for (parts are bound
        one after the other, so such a source keeps peak memory at the model plus one part)."""
        def local_view(part: Part) -> dict[str, torch.Tensor]:
            return {local: tensors[part.spec.tensor_name(local)] for local in part.param_decls()}

        self.embedding.bind(local_view(self.embedding), dtype, device)
        for b in self.blocks:
            for part in b.parts():
                part.bind(local_view(part), dtype, device)
        self.final_norm.bind(local_view(self.final_norm), dtype, device)
        if getattr(self.head, "tied", False):
            self.head.bind({}, dtype, device, tied_weight=self.embedding.weight)
        else:
            self.head.bind(local_view(self.head), dtype, device)
        self.dtype, self.device = dtype, device
        self._bound = True

    # ------------------------------------------------------------------ one step

    def forward(self, ctx: StepContext, caches: list[LayerCache], want_rows: torch.Tensor | None,
                n_want: int) -> torch.Tensor:
        """fp32 logits ``[n_want, vocab]`` at the packed rows ``want_rows`` (int32)."""
        if not self._bound:
            raise RuntimeError("the model has no weights yet")
        x = self.embedding.forward(ctx)
        residual = None
        for i, (entry, cache) in enumerate(zip(self.schedule, caches)):
            block = self.blocks[entry.layer]
            if block.entry() is None:
                x, residual = block.forward(x, residual, ctx, cache)
                continue
            # a layer that takes part in the hand-over of norms is told how the next one begins
            after = self.blocks[self.schedule[i + 1].layer].entry() if i + 1 < len(self.schedule) else None
            x, residual = block.forward(x, residual, ctx, cache, following=after)
        if n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        z, _ = self.final_norm.forward(x, residual, rows=want_rows)
        return self.head.forward(z)
