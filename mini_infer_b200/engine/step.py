"""The step function: one batch of (request, its next tokens) through the model.

``StepRunner.step(entries)`` takes any mix of prompt portions and single decoded tokens,
cut anywhere.  It plans on the host first (positions come from the cache's own lengths,
pages are reserved for every request of the step or ``OutOfPages`` is raised with nothing
changed), uploads one descriptor buffer (the batch's lists and the page ids handed out
since the last step; the block tables themselves stay on the device), runs the model on
exactly the tokens it was given, reading everything older from the cache, and returns fp32
logits at the wanted places only.  The reference's counterpart is ``ModelRunner.forward_step_packed``
(``engine/model_runner.py:270-395``), which reserves pages inside the forward pass instead.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
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

    device_buffer: torch.Tensor       # int32 descriptors at fixed addresses
    graph: "torch.cuda.CUDAGraph | None" = None
    logits: torch.Tensor | None = None
    replays: int = 0
    launches: int = 0                 # kernels recorded in the graph


@dataclass
class HostPlan:
    """A step's descriptors on the host: one int32 buffer and where each list lies in it."""

    buffer: np.ndarray
    offsets: dict[str, tuple[int, int]]
    n_tokens: int
    q_start: list[int]
    q_len: list[int]
    kv_len: list[int]
    state_slots: list[int]
    rows: list[tuple[Hashable, int]]
    decode_only: bool
    update_capacity: list[int]         # per group: triples the buffer has room for
    overflow: list[list[int]]          # per group: triples that did not fit a captured step's fixed room
    tile_counts: dict[int, int]
    n_single: int = 0                  # a mixed step's requests that bring one token
    multi_counts: dict[int, int] = field(default_factory=dict)   # tiles of the others, per tile size


class StepRunner:
    """``cuda_graph=True`` replays decode-only steps (every request brings one token and
    wants its logits) as captured CUDA graphs, one per batch size (the lengths, the pages and
    how decode attention spreads its keys over blocks are all read from device memory when the
    graph runs); the reference keeps such graphs per batch bucket (``engine/paged_decode_graph.py:67-225``).
    Everything else runs kernel by kernel, and so does every step of a model one of whose parts
    is not ``graph_safe``.

    The block tables live on the device (``CacheManager.block_tables``); a step uploads only
    the page ids the host has just handed out and scatters them in before its first kernel,
    so what a step copies to the device does not grow with the context."""

    def __init__(self, model: DecoderModel, cache: CacheManager, cuda_graph: bool = False) -> None:
        self.model = model
        self.cache = cache
        self.cuda_graph = cuda_graph and model.graph_safe()
        self._graphs: dict[tuple, GraphSlot] = {}
        self._layer_caches: list[LayerCache] | None = None
        self.device = model.device
        self.dtype = model.dtype
        self.vocab_size = model.spec.vocab_size
        needs = model.plan_needs()
        self.tile_sizes = sorted(needs.q_tile_tokens)
        self.max_positions = model.spec.max_positions
        self.sm_count = ops.sm_count(self.device) if self.device is not None and self.device.type == "cuda" else 148
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

    def host_plan(self, entries: Sequence[StepEntry], graphed: bool = False) -> HostPlan:
        """Reserve pages and lay the step's descriptors out in one host buffer (no device work).

        With ``graphed`` the layout depends only on the batch size: every list has a fixed
        length (one token per request, room for one new page per request and group)."""
        self._validate(entries)
        plan: AppendPlan = self.cache.plan_append([(e.rid, len(e.tokens)) for e in entries])
        updates = self.cache.take_table_updates()
        B = len(entries)
        q_len = plan.counts
        q_start = [0] * B
        for i in range(1, B):
            q_start[i] = q_start[i - 1] + q_len[i - 1]
        M = q_start[-1] + q_len[-1]
        kv_len = [s + n for s, n in zip(plan.start, plan.counts)]
        decode_only = M == B
        want_rows: list[int] = []
        rows: list[tuple[Hashable, int]] = []
        if decode_only:
            tokens = [int(e.tokens[0]) for e in entries]
            positions = plan.start
            for i, e in enumerate(entries):
                for w in e.want:
                    want_rows.append(i)
                    rows.append((e.rid, int(w)))
        else:
            tokens, positions = [], []
            for i, e in enumerate(entries):
                tokens.extend(int(t) for t in e.tokens)
                positions.extend(range(plan.start[i], kv_len[i]))
                for w in e.want:
                    want_rows.append(q_start[i] + int(w))
                    rows.append((e.rid, int(w)))

        parts: list[tuple[str, Sequence[int]]] = [
            ("token_ids", tokens), ("positions", positions), ("q_start", q_start),
            ("q_len", q_len), ("kv_len", kv_len), ("state_slot", plan.state_slots),
            ("want_rows", want_rows),
        ]
        n_groups = len(self.cache.groups)
        capacity, overflow = [0] * n_groups, [[] for _ in range(n_groups)]
        for gi, g in enumerate(self.cache.groups):
            parts.append((f"slots{gi}", plan.token_slots[gi]))
            flat = updates[gi]
            if graphed:
                capacity[gi] = B
                if len(flat) > 3 * B:      # pages handed out outside a step (rare): sent separately
                    overflow[gi], flat = flat, []
                parts.append((f"updates{gi}", list(flat) + [-1] * (3 * B - len(flat))))
            else:
                capacity[gi] = len(flat) // 3
                parts.append((f"updates{gi}", flat))
            parts.append((f"update_count{gi}", [len(flat) // 3]))
        # In a mixed step the requests that bring a single token can go to the decode kernel,
        # which spreads their keys over all blocks (as one tile of the prefill kernels such a
        # request is one block per head group walking its whole context alone); the tiles of the
        # others are listed a second time without them.
        singles = [] if decode_only else [i for i in range(B) if q_len[i] == 1]
        if len(singles) == B:
            singles = []
        parts.append(("single_q_start", [q_start[i] for i in singles]))
        parts.append(("single_kv_len", [kv_len[i] for i in singles]))
        parts.append(("single_rows", [plan.state_slots[i] for i in singles]))
        tile_counts: dict[int, int] = {}
        multi_counts: dict[int, int] = {}
        for n in self.tile_sizes:
            if decode_only:
                treq: Sequence[int] = range(B)
                ttok: Sequence[int] = [0] * B
            else:
                # Tiles with the most keys to walk come first: the attention kernels start their
                # blocks in this order, so the long ones are under way when the short ones fill
                # what is left (a tile of tokens t0.. of request i sees its keys up to the tile's end).
                tiles = [(i, t0) for i in range(B) for t0 in range(0, q_len[i], n)]
                tiles.sort(key=lambda it: -(kv_len[it[0]] - q_len[it[0]] + min(q_len[it[0]], it[1] + n)))
                treq = [i for i, _ in tiles]
                ttok = [t0 for _, t0 in tiles]
            tile_counts[n] = len(treq)
            parts.append((f"tile_req{n}", treq))
            parts.append((f"tile_tok{n}", ttok))
            if singles:
                keep = [j for j, i in enumerate(treq) if q_len[i] > 1]
                multi_counts[n] = len(keep)
                parts.append((f"multi_req{n}", [treq[j] for j in keep]))
                parts.append((f"multi_tok{n}", [ttok[j] for j in keep]))

        offsets: dict[str, tuple[int, int]] = {}
        total = 0
        for name, lst in parts:
            offsets[name] = (total, len(lst))
            total += (len(lst) + 3) // 4 * 4      # keep every slice 16-byte aligned
        buffer = np.empty(max(total, 4), dtype=np.int32)
        for name, lst in parts:
            o, n = offsets[name]
            if n:
                buffer[o:o + n] = lst
        return HostPlan(buffer=buffer, offsets=offsets, n_tokens=M, q_start=q_start, q_len=list(q_len),
                        kv_len=kv_len, state_slots=list(plan.state_slots), rows=rows, decode_only=decode_only,
                        update_capacity=capacity, overflow=overflow, tile_counts=tile_counts,
                        n_single=len(singles), multi_counts=multi_counts)

    def plan(self, entries: Sequence[StepEntry], graphed: bool = False):
        """Reserve pages and put the step's descriptors on the device (one copy).

        With ``graphed`` the descriptors are copied into the fixed device buffer of the
        matching ``GraphSlot``, which is returned as a fifth value."""
        hp = self.host_plan(entries, graphed)
        B = len(entries)
        host = torch.empty(hp.buffer.shape[0], dtype=torch.int32, pin_memory=True)
        host.numpy()[:] = hp.buffer
        slot = None
        if graphed:
            key = (B,)
            slot = self._graphs.get(key)
            if slot is None:
                slot = GraphSlot(device_buffer=torch.empty(host.numel(), dtype=torch.int32, device=self.device))
                self._graphs[key] = slot
            dev = slot.device_buffer
            dev.copy_(host, non_blocking=True)
        else:
            dev = host.to(self.device, non_blocking=True)
        self.last_h2d_bytes = host.numel() * 4
        for gi, flat in enumerate(hp.overflow):
            if flat:
                extra = torch.tensor(flat + [len(flat) // 3], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
                self.last_h2d_bytes += extra.numel() * 4
                ops.table_update(self.cache.block_tables[gi], extra, extra[len(flat):], len(flat) // 3)

        def view(name: str) -> torch.Tensor:
            o, n = hp.offsets[name]
            return dev[o:o + n]

        groups = []
        state_slot = view("state_slot")
        for gi, g in enumerate(self.cache.groups):
            groups.append(GroupView(
                page_size=self.cache.page_size, window=g.window,
                block_table=self.cache.block_tables[gi], slots=view(f"slots{gi}"), table_rows=state_slot,
            ))
        ctx = StepContext(
            dtype=self.dtype, device=self.device, n_tokens=hp.n_tokens, n_requests=B,
            token_ids=view("token_ids"), positions=view("positions"), q_start=view("q_start"),
            q_len=view("q_len"), kv_len=view("kv_len"), state_slot=state_slot,
            host_q_start=hp.q_start, host_q_len=hp.q_len, host_kv_len=hp.kv_len,
            host_state_slot=hp.state_slots, groups=groups,
            tiles={n: (view(f"tile_req{n}"), view(f"tile_tok{n}"), hp.tile_counts[n]) for n in self.tile_sizes},
            decode_only=hp.decode_only,
            n_single=hp.n_single,
            single_q_start=view("single_q_start"), single_kv_len=view("single_kv_len"), single_rows=view("single_rows"),
            tiles_multi={n: (view(f"multi_req{n}"), view(f"multi_tok{n}"), hp.multi_counts[n]) for n in hp.multi_counts},
            # a captured step must not depend on the lengths of the day: it is planned for
            # the longest context its block tables can hold
            max_kv_len=(max(self.cache.table_width, default=1) * self.cache.page_size) if graphed else max(hp.kv_len),
        )
        ctx.table_updates = [(view(f"updates{gi}"), view(f"update_count{gi}"), hp.update_capacity[gi])
                             for gi in range(len(self.cache.groups))]
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
        want = view("want_rows") if hp.rows else None
        if graphed:
            return ctx, caches, want, hp.rows, slot
        return ctx, caches, want, hp.rows

    # ------------------------------------------------------------------ running

    def _graphable(self, entries: Sequence[StepEntry]) -> bool:
        return self.cuda_graph and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    def apply_table_updates(self, ctx: StepContext) -> None:
        """Scatter the page ids a planned step brought along into the device block tables.
        ``step`` does this itself; a caller that plans a step and runs parts by hand calls it
        before the first kernel that reads a block table."""
        for gi, (updates, count, capacity) in enumerate(ctx.table_updates):
            if capacity:
                ops.table_update(self.cache.block_tables[gi], updates, count, capacity)

    def _run(self, ctx: StepContext, caches, want, n_want: int) -> torch.Tensor:
        """The device work of a step: the new page ids into the block tables, then the model."""
        ctx.scratch.clear()   # what the parts share within a step is made anew in every run (and in a capture)
        self.apply_table_updates(ctx)
        return self.model.forward(ctx, caches, want, n_want)

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
        logits = self._run(ctx, caches, want, len(rows))
        self.steps_run += 1
        return StepResult(logits=logits, rows=rows)

    def _graphed_step(self, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None = None) -> StepResult:
        """Replay the CUDA graph of a decode-only step.  The first step of a kind runs kernel by
        kernel (that is the step itself: every kernel gets compiled and configured, and the
        step's effects happen once) and is then captured, without being run again, for the
        steps that follow.  A replayed step's logits live in the graph's own memory and are
        overwritten by the next replay of the same graph."""
        ctx, caches, want, rows, slot = self.plan(entries, graphed=True)
        if device_tokens is not None:
            ctx.token_ids.copy_(device_tokens)   # into the graph's fixed descriptor buffer
        if slot.graph is None:
            logits = self._run(ctx, caches, want, len(rows))
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with torch.cuda.graph(graph):       # records the launches; nothing runs
                slot.logits = self._run(ctx, caches, want, len(rows))
            slot.launches = ops.launch_count - before
            ops.launch_count = before           # the capture launched nothing
            slot.graph = graph
            self.steps_run += 1
            return StepResult(logits=logits, rows=rows)
        slot.graph.replay()
        ops.launch_count += slot.launches
        slot.replays += 1
        self.steps_run += 1
        return StepResult(logits=slot.logits, rows=rows)
