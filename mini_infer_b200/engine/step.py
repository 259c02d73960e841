"""The step function: one batch of (request, its next tokens) through the model.

``StepRunner.step(entries)`` takes any mix of prompt portions and single decoded tokens,
cut anywhere.  It plans on the host first (positions come from the cache's own lengths,
pages are reserved for every request of the step or ``OutOfPages`` is raised with nothing
changed), uploads one descriptor buffer, runs the model on exactly the tokens it was
given, reading everything older from the cache, and returns fp32 logits at the wanted
places only.  The reference's counterpart is ``ModelRunner.forward_step_packed``
(``engine/model_runner.py:270-395``), which reserves pages inside the forward pass instead.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import torch

from ..cache.manager import AppendPlan, CacheManager
from ..parts.base import GroupView, LayerCache, StepContext
from ..parts.model import DecoderModel


class StepError(ValueError):
    pass


@dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens`` and the places (indices into
    ``tokens``) whose logits are wanted (may be empty)."""

    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


@dataclass
class StepResult:
    logits: torch.Tensor            # [n_wanted, vocab] fp32, in the order of entries and of want
    rows: list[tuple[Hashable, int]]  # (request, index within its tokens) of every logits row


class StepRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager) -> None:
        self.model = model
        self.cache = cache
        self.device = model.device
        self.dtype = model.dtype
        self.vocab_size = model.spec.vocab_size
        self.tile_sizes = sorted(model.plan_needs().q_tile_tokens)
        self.max_positions = model.spec.max_positions
        self.steps_run = 0
        self.last_h2d_bytes = 0

    # ------------------------------------------------------------------ planning

    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        V = self.vocab_size
        for e in entries:
            if len(e.tokens) == 0:
                raise StepError(f"request {e.rid!r}: no tokens in this step")
            for t in e.tokens:
                if not 0 <= int(t) < V:
                    raise StepError(f"request {e.rid!r}: token id {t} is outside [0, {V})")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise StepError(f"request {e.rid!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
            if self.max_positions is not None and e.rid in self.cache:
                if self.cache.length(e.rid) + len(e.tokens) > self.max_positions:
                    raise StepError(
                        f"request {e.rid!r} would pass the model's {self.max_positions} positions"
                    )

    def plan(self, entries: Sequence[StepEntry]) -> tuple[StepContext, list[LayerCache], torch.Tensor | None, list]:
        """Reserve pages and build the step's descriptors on the device."""
        self._validate(entries)
        plan: AppendPlan = self.cache.plan_append([(e.rid, len(e.tokens)) for e in entries])
        B = len(entries)
        q_len = plan.counts
        q_start = [0] * B
        for i in range(1, B):
            q_start[i] = q_start[i - 1] + q_len[i - 1]
        M = q_start[-1] + q_len[-1]
        kv_len = [s + n for s, n in zip(plan.start, plan.counts)]
        tokens: list[int] = []
        positions: list[int] = []
        want_rows: list[int] = []
        rows: list[tuple[Hashable, int]] = []
        for i, e in enumerate(entries):
            tokens.extend(int(t) for t in e.tokens)
            positions.extend(range(plan.start[i], kv_len[i]))
            for w in e.want:
                want_rows.append(q_start[i] + int(w))
                rows.append((e.rid, int(w)))

        # one staging buffer: every list becomes a slice of it
        parts: list[tuple[str, list[int]]] = [
            ("token_ids", tokens), ("positions", positions), ("q_start", q_start),
            ("q_len", q_len), ("kv_len", kv_len), ("state_slot", plan.state_slots),
            ("want_rows", want_rows),
        ]
        widths: list[int] = []
        for gi in range(len(self.cache.groups)):
            width = max(1, max(len(t) for t in plan.tables[gi]))
            widths.append(width)
            flat: list[int] = []
            for t in plan.tables[gi]:
                flat.extend(t)
                flat.extend([-1] * (width - len(t)))
            parts.append((f"table{gi}", flat))
            parts.append((f"slots{gi}", plan.token_slots[gi]))
        tile_counts: dict[int, int] = {}
        for n in self.tile_sizes:
            treq: list[int] = []
            ttok: list[int] = []
            for i in range(B):
                for t0 in range(0, q_len[i], n):
                    treq.append(i)
                    ttok.append(t0)
            tile_counts[n] = len(treq)
            parts.append((f"tile_req{n}", treq))
            parts.append((f"tile_tok{n}", ttok))

        offsets: dict[str, tuple[int, int]] = {}
        total = 0
        for name, lst in parts:
            offsets[name] = (total, len(lst))
            total += (len(lst) + 3) // 4 * 4      # keep every slice 16-byte aligned
        host = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=True)
        host_np = host.numpy()
        for name, lst in parts:
            o, n = offsets[name]
            if n:
                host_np[o:o + n] = lst
        dev = host.to(self.device, non_blocking=True)
        self.last_h2d_bytes = host.numel() * 4

        def view(name: str) -> torch.Tensor:
            o, n = offsets[name]
            return dev[o:o + n]

        groups = []
        for gi, g in enumerate(self.cache.groups):
            groups.append(GroupView(
                page_size=self.cache.page_size, window=g.window,
                block_table=view(f"table{gi}").view(B, widths[gi]), slots=view(f"slots{gi}"),
            ))
        ctx = StepContext(
            dtype=self.dtype, device=self.device, n_tokens=M, n_requests=B,
            token_ids=view("token_ids"), positions=view("positions"), q_start=view("q_start"),
            q_len=view("q_len"), kv_len=view("kv_len"), state_slot=view("state_slot"),
            host_q_start=q_start, host_q_len=list(q_len), host_kv_len=kv_len,
            host_state_slot=list(plan.state_slots), groups=groups,
            tiles={n: (view(f"tile_req{n}"), view(f"tile_tok{n}"), tile_counts[n]) for n in self.tile_sizes},
            decode_only=all(n == 1 for n in q_len), max_kv_len=max(kv_len),
        )
        caches: list[LayerCache] = []
        for entry in self.model.schedule:
            lc = LayerCache(writes=entry.writes_cache)
            if entry.cache in self.cache.layer_place:
                lc.group, lc.k, lc.v = self.cache.layer_kv(entry.cache)
            lc.state = self.cache.layer_state(entry.cache)
            caches.append(lc)
        want = view("want_rows") if want_rows else None
        return ctx, caches, want, rows

    # ------------------------------------------------------------------ running

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> StepResult:
        ctx, caches, want, rows = self.plan(entries)
        logits = self.model.forward(ctx, caches, want, len(rows))
        self.steps_run += 1
        return StepResult(logits=logits, rows=rows)
