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
from ..csrc import ops
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


@dataclass
class GraphSlot:
    """A captured decode step: the CUDA graph, its fixed descriptor buffer and its logits."""

    widths: list[int]                 # block-table width (pages) per cache group
    device_buffer: torch.Tensor       # int32 descriptors at fixed addresses
    graph: "torch.cuda.CUDAGraph | None" = None
    logits: torch.Tensor | None = None
    ctx: StepContext | None = None
    replays: int = 0
    launches: int = 0                 # kernels recorded in the graph


class StepRunner:
    """``cuda_graph=True`` replays decode-only steps (every request brings one token and
    wants its logits) as captured CUDA graphs, one per (batch size, block-table width
    bucket, number of key slices); the reference keeps such graphs per batch bucket
    (``engine/paged_decode_graph.py:67-225``).  Everything else runs kernel by kernel."""

    GRAPH_WIDTH_BUCKET = 64           # block tables of a captured step grow in steps of 64 pages

    def __init__(self, model: DecoderModel, cache: CacheManager, cuda_graph: bool = False) -> None:
        self.model = model
        self.cache = cache
        self.cuda_graph = cuda_graph
        self._graphs: dict[tuple, GraphSlot] = {}
        self._layer_caches: list[LayerCache] | None = None
        self.device = model.device
        self.dtype = model.dtype
        self.vocab_size = model.spec.vocab_size
        needs = model.plan_needs()
        self.tile_sizes = sorted(needs.q_tile_tokens)
        self.decode_blocks_per_request = needs.decode_blocks_per_request
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

    def plan(self, entries: Sequence[StepEntry], graphed: bool = False):
        """Reserve pages and build the step's descriptors on the device.

        With ``graphed`` the descriptors get a layout that depends only on the batch size
        and the (bucketed) block-table widths, and are copied into that layout's fixed
        device buffer; the matching ``GraphSlot`` is returned as a fifth value."""
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
            if graphed:
                width = -(-width // self.GRAPH_WIDTH_BUCKET) * self.GRAPH_WIDTH_BUCKET
            widths.append(width)
            flat: list[int] = []
            for t in plan.tables[gi]:
                flat.extend(t)
                flat.extend([-1] * (width - len(t)))
            parts.append((f"table{gi}", flat))
            parts.append((f"slots{gi}", plan.token_slots[gi]))
        # Decode-only steps of a mixer that cuts keys into slices: how many, and how long
        # (one int per group on the device, so that a captured step follows the lengths).
        decode_only = all(n == 1 for n in q_len)
        slices: list[int] = [0] * len(self.cache.groups)
        if decode_only and self.decode_blocks_per_request > 0 and self.dtype == torch.bfloat16:
            for gi, g in enumerate(self.cache.groups):
                slices[gi], per = ops.decode_plan(kv_len, g.window or 0, self.decode_blocks_per_request,
                                                  ops.sm_count(self.device))
                parts.append((f"slice{gi}", [per]))
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
        slot = None
        if graphed:
            key = (B, tuple(widths), tuple(slices))
            slot = self._graphs.get(key)
            if slot is None:
                slot = GraphSlot(widths=list(widths),
                                 device_buffer=torch.empty(host.numel(), dtype=torch.int32, device=self.device))
                self._graphs[key] = slot
            dev = slot.device_buffer
            dev.copy_(host, non_blocking=True)
        else:
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
                decode_slices=slices[gi], decode_slice_chunks=view(f"slice{gi}") if slices[gi] else None,
            ))
        ctx = StepContext(
            dtype=self.dtype, device=self.device, n_tokens=M, n_requests=B,
            token_ids=view("token_ids"), positions=view("positions"), q_start=view("q_start"),
            q_len=view("q_len"), kv_len=view("kv_len"), state_slot=view("state_slot"),
            host_q_start=q_start, host_q_len=list(q_len), host_kv_len=kv_len,
            host_state_slot=list(plan.state_slots), groups=groups,
            tiles={n: (view(f"tile_req{n}"), view(f"tile_tok{n}"), tile_counts[n]) for n in self.tile_sizes},
            decode_only=decode_only,
            # a captured step must not depend on the lengths of the day: it is planned for
            # the longest context its block tables can hold
            max_kv_len=(max(widths) * self.cache.page_size) if graphed else max(kv_len),
        )
        if self._layer_caches is None:     # the views never change: build them once
            caches: list[LayerCache] = []
            for entry in self.model.schedule:
                lc = LayerCache(writes=entry.writes_cache)
                if entry.cache in self.cache.layer_place:
                    lc.group, lc.k, lc.v = self.cache.layer_kv(entry.cache)
                lc.state = self.cache.layer_state(entry.cache)
                caches.append(lc)
            self._layer_caches = caches
        caches = self._layer_caches
        want = view("want_rows") if want_rows else None
        if graphed:
            return ctx, caches, want, rows, slot
        return ctx, caches, want, rows

    # ------------------------------------------------------------------ running

    def _graphable(self, entries: Sequence[StepEntry]) -> bool:
        return self.cuda_graph and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None = None) -> StepResult:
        """Run one batch.  ``device_tokens`` (int32 on the device, one per entry) replaces the
        entries' token ids for a step whose every entry brings exactly one token: the ids are
        then taken from that tensor on the device, in stream order, and the ids in ``entries``
        are placeholders.  A scheduler uses it to launch the next decode step from the
        sampler's output before the host has seen it."""
        if device_tokens is not None:
            if any(len(e.tokens) != 1 for e in entries):
                raise StepError("device_tokens needs entries of exactly one token each")
            if (device_tokens.dtype != torch.int32 or device_tokens.shape != (len(entries),)
                    or device_tokens.device != self.device):
                raise StepError("device_tokens must be an int32 vector on the model's device, one per entry")
        if self._graphable(entries):
            return self._graphed_step(entries, device_tokens)
        ctx, caches, want, rows = self.plan(entries)
        if device_tokens is not None:
            ctx.token_ids.copy_(device_tokens)
        logits = self.model.forward(ctx, caches, want, len(rows))
        self.steps_run += 1
        return StepResult(logits=logits, rows=rows)

    def _graphed_step(self, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None = None) -> StepResult:
        """Replay (first: capture) the CUDA graph of a decode-only step.  The logits live in
        the graph's own memory and are overwritten by the next replay of the same graph."""
        ctx, caches, want, rows, slot = self.plan(entries, graphed=True)
        if device_tokens is not None:
            ctx.token_ids.copy_(device_tokens)   # into the graph's fixed descriptor buffer
        if slot.graph is None:
            # run once kernel by kernel (compiles and configures every kernel), then capture
            # the same launches; both read the descriptors just copied into the fixed buffer
            # and write this step's keys and values to the same slots, so repeating is harmless
            self.model.forward(ctx, caches, want, len(rows))
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with torch.cuda.graph(graph):
                slot.logits = self.model.forward(ctx, caches, want, len(rows))
            slot.launches = ops.launch_count - before
            ops.launch_count = before
            slot.graph, slot.ctx = graph, ctx
        slot.graph.replay()
        ops.launch_count += slot.launches
        slot.replays += 1
        self.steps_run += 1
        return StepResult(logits=slot.logits, rows=rows)
