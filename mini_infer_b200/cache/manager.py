"""The cache manager: pages of keys and values, block tables, and fixed-size state slots.

*Groups.*  Cache layers whose mixers keep the same thing (key/value heads, head size,
window) form a group.  A group owns its pages: a pool of page ids with a LIFO free
list, one storage tensor ``[layers, 2, pages, kv_heads, page_size, head_dim]`` (the keys of a
page lie together per head, so attention reads long runs) and one
block table per request.  A page id means the same row range in every layer of its group
(the reference's pool works that way for its single group, ``cache/block_pool.py:332-351``;
its free list is LIFO as well, ``:570,735-757``).  Groups with a window give pages back as
soon as every position in them has fallen out of every future query's window; the table
keeps ``-1`` there, and kernels never look below the window.

*Requests.*  ``add_request`` hands out a stable slot (requests never move when another one
ends, unlike the reference's ``remove_request`` which shifts indices,
``cache/paged_kv_cache.py:245-258``).  ``plan_append`` reserves room for a step's new tokens
for all requests of the step at once, before anything is launched: either every page is
there and the plan is returned, or ``OutOfPages`` is raised and nothing has changed.
``free_request`` returns everything.

*Block tables on the device.*  Each group has one int32 table ``[max_requests, table_width]``
on the device, a row per request slot.  The host keeps the authoritative tables; a plan
records only the pages it has just handed out as ``(slot, index, page)`` triples, which the
step uploads with its descriptors and scatters into the device table before its first kernel
reads it.  What a step sends to the device therefore does not grow with the context.  Entries
of pages that a window has given back are left as they are: no kernel looks below a window.

*State slots.*  A mixer with a per-request state of fixed size gets an arena
``[max_requests, *shape]`` per cache layer; a request's row is its slot, zeroed on
admission.  Llama has no such state; the arena exists for mixers that do.

All bookkeeping is host-side Python over plain lists and can be used (and is tested)
without a GPU by passing ``device=None``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Iterable, Sequence

import torch


class OutOfPages(RuntimeError):
    """Not enough free pages for what was asked; nothing was changed."""


class CacheError(RuntimeError):
    pass


class PagePool:
    """Page ids ``0 .. num_pages-1`` with a LIFO free list."""

    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise CacheError(f"a pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # pop() hands out 0 first
        self._is_free = [True] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        self._is_free[page] = False
        return page

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page {page} is not in the pool")
        if self._is_free[page]:
            raise CacheError(f"page {page} is freed twice")
        self._is_free[page] = True
        self._free.append(page)

    def free_pages(self) -> list[int]:
        return list(self._free)


@dataclass(frozen=True)
class GroupSpec:
    layers: tuple[int, ...]        # cache layer indices of this group
    kv_heads: int
    head_dim: int
    window: int | None


@dataclass
class _Request:
    rid: Hashable
    slot: int
    length: int = 0                                  # tokens held
    tables: list[list[int]] = field(default_factory=list)   # per group: page ids, -1 = given back
    released: list[int] = field(default_factory=list)       # per group: leading pages given back


@dataclass
class AppendPlan:
    """Where a step's new tokens go.  Lists are in the order of the step's entries."""

    rids: list[Hashable]
    state_slots: list[int]
    start: list[int]                     # tokens held before the step, per request
    counts: list[int]                    # new tokens per request
    token_slots: list[list[int]]         # per group: flat slot of every new token (all requests)


def group_needs(needs: Sequence) -> list[GroupSpec]:
    """Partition cache layers by what they keep per token."""
    order: list[tuple] = []
    members: dict[tuple, list[int]] = {}
    for n in needs:
        if n.kv is None:
            continue
        key = (n.kv.kv_heads, n.kv.head_dim, n.kv.window)
        if key not in members:
            members[key] = []
            order.append(key)
        members[key].append(n.index)
    return [GroupSpec(tuple(members[k]), k[0], k[1], k[2]) for k in order]


class CacheManager:
    def __init__(
        self,
        needs: Sequence,
        *,
        page_size: int,
        num_pages: int | Sequence[int],
        max_requests: int,
        dtype: torch.dtype = torch.bfloat16,
        device: torch.device | str | None = None,
        max_request_tokens: int | None = None,
    ) -> None:
        if page_size <= 0:
            raise CacheError(f"page size must be positive, got {page_size}")
        if max_requests <= 0:
            raise CacheError(f"max_requests must be positive, got {max_requests}")
        self.page_size = page_size
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.needs = list(needs)
        self.groups = group_needs(self.needs)
        if isinstance(num_pages, int):
            pages = [num_pages] * len(self.groups)
        else:
            pages = list(num_pages)
            if len(pages) != len(self.groups):
                raise CacheError(f"{len(self.groups)} groups but {len(pages)} page counts")
        self.pools = [PagePool(n) for n in pages]
        self._windowed = [gi for gi, g in enumerate(self.groups) if g.window is not None]
        self._requests: dict[Hashable, _Request] = {}
        self._free_slots = list(range(max_requests - 1, -1, -1))

        # cache layer -> (group index, index within the group's storage)
        self.layer_place: dict[int, tuple[int, int]] = {}
        for gi, g in enumerate(self.groups):
            for li, layer in enumerate(g.layers):
                self.layer_place[layer] = (gi, li)

        # Width of a request's block table: no request holds more pages than its group's pool
        # has, nor more than the longest sequence the caller allows.
        # (A windowed group hands pages back, so its requests may be longer than its pool: its
        # tables are as wide as the longest sequence, 65,536 pages when the caller names none.)
        cap = None if max_request_tokens is None else -(-int(max_request_tokens) // page_size)
        self.table_width = []
        for g, n in zip(self.groups, pages):
            widest = n if g.window is None else max(n, 65536 if cap is None else cap)
            self.table_width.append(max(1, widest if cap is None else min(widest, cap)))
        # pages handed out since the last take_table_updates(): flat (slot, index, page) triples
        self._table_updates: list[list[int]] = [[] for _ in self.groups]

        self.storage: list[torch.Tensor] = []
        self.block_tables: list[torch.Tensor] = []
        self.state_arenas: dict[int, torch.Tensor] = {}
        if self.device is not None:
            for g, n, width in zip(self.groups, pages, self.table_width):
                self.storage.append(
                    torch.zeros((len(g.layers), 2, n, g.kv_heads, page_size, g.head_dim),
                                dtype=dtype, device=self.device)
                )
                self.block_tables.append(torch.full((max_requests, width), -1, dtype=torch.int32, device=self.device))
            for need in self.needs:
                if need.state is not None:
                    self.state_arenas[need.index] = torch.zeros(
                        (max_requests, *need.state.shape), dtype=need.state.dtype, device=self.device
                    )
        self._has_state = any(n.state is not None for n in self.needs)

    # ------------------------------------------------------------------ requests

    def __contains__(self, rid: Hashable) -> bool:
        return rid in self._requests

    @property
    def num_requests(self) -> int:
        return len(self._requests)

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def length(self, rid: Hashable) -> int:
        return self._get(rid).length

    def slot(self, rid: Hashable) -> int:
        return self._get(rid).slot

    def table(self, rid: Hashable, group: int = 0) -> list[int]:
        """A copy of a request's block table in ``group`` (page ids; -1 where a window gave
        the page back)."""
        return list(self._get(rid).tables[group])

    def take_table_updates(self) -> list[list[int]]:
        """Per group, the ``(slot, index, page)`` triples (flat) of every page handed out since
        the last call, in the order they were handed out.  Whoever runs steps on the device
        must scatter them into ``block_tables`` before the step's kernels run."""
        out = self._table_updates
        self._table_updates = [[] for _ in self.groups]
        return out

    def _get(self, rid: Hashable) -> _Request:
        try:
            return self._requests[rid]
        except KeyError:
            raise CacheError(f"unknown request {rid!r}") from None

    def add_request(self, rid: Hashable) -> int:
        """Admit a request: a slot of its own, empty block tables, zeroed state."""
        if rid in self._requests:
            raise CacheError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        self._requests[rid] = _Request(
            rid, slot, 0, [[] for _ in self.groups], [0 for _ in self.groups]
        )
        for arena in self.state_arenas.values():
            arena[slot].zero_()
        return slot

    def free_request(self, rid: Hashable) -> None:
        """Give back every page and the slot of a finished (or preempted) request."""
        req = self._get(rid)
        for gi, table in enumerate(req.tables):
            for page in table:
                if page >= 0:
                    self.pools[gi].free(page)
        del self._requests[rid]
        self._free_slots.append(req.slot)

    # ------------------------------------------------------------------ pages

    def _window_release_count(self, gi: int, length: int) -> int:
        """Leading pages of a request holding ``length`` tokens that no future query reads."""
        w = self.groups[gi].window
        if w is None:
            return 0
        first_needed = length - w + 1      # the next query sits at position >= length
        if first_needed <= 0:
            return 0
        return first_needed // self.page_size

    def pages_needed(self, entries: Iterable[tuple[Hashable, int]]) -> list[int]:
        """Pages each group must still hand out for these ``(request, new tokens)``,
        counting the pages a windowed group gets back first."""
        need = [0] * len(self.groups)
        for rid, n_new in entries:
            req = self._get(rid)
            want = -(-(req.length + n_new) // self.page_size)
            for gi, g in enumerate(self.groups):
                need[gi] += max(0, want - len(req.tables[gi]))
                if g.window is not None:
                    need[gi] -= max(0, self._window_release_count(gi, req.length) - req.released[gi])
        return need

    def can_append(self, entries: Iterable[tuple[Hashable, int]]) -> bool:
        entries = list(entries)
        return all(n <= pool.num_free for n, pool in zip(self.pages_needed(entries), self.pools))

    def plan_append(self, entries: Sequence[tuple[Hashable, int]]) -> AppendPlan:
        """Reserve room for ``n_new`` tokens of each request; all or nothing."""
        seen = set()
        for rid, n_new in entries:
            if n_new <= 0:
                raise CacheError(f"request {rid!r}: a step must bring at least one token")
            if rid in seen:
                raise CacheError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
            self._get(rid)
        need = self.pages_needed(entries)
        for gi, (n, pool) in enumerate(zip(need, self.pools)):
            if n > pool.num_free:
                raise OutOfPages(
                    f"group {gi} needs {n} more pages, {pool.num_free} of {pool.num_pages} are free"
                )
        room = min(self.table_width, default=0) * self.page_size
        for rid, n_new in entries:
            if self.groups and self._requests[rid].length + n_new > room:
                raise CacheError(
                    f"request {rid!r} would hold {self._requests[rid].length + n_new} tokens; a block table "
                    f"takes {room}"
                )
        plan = AppendPlan([], [], [], [], [[] for _ in self.groups])
        ps = self.page_size
        # pages that have fallen out of a window go back first, for every request of the
        # step, so that the allocations below may use them
        for rid, _ in entries if self._windowed else ():
            req = self._requests[rid]
            for gi in self._windowed:
                pool = self.pools[gi]
                table = req.tables[gi]
                upto = min(self._window_release_count(gi, req.length), len(table))
                for idx in range(req.released[gi], upto):
                    if table[idx] >= 0:
                        pool.free(table[idx])
                        table[idx] = -1
                req.released[gi] = max(req.released[gi], upto)
        for rid, n_new in entries:
            req = self._requests[rid]
            start, total = req.length, req.length + n_new
            plan.rids.append(rid)
            plan.state_slots.append(req.slot)
            plan.start.append(start)
            plan.counts.append(n_new)
            for gi, pool in enumerate(self.pools):
                table = req.tables[gi]
                updates = self._table_updates[gi]
                while len(table) * ps < total:
                    page = pool.allocate()
                    updates.extend((req.slot, len(table), page))
                    table.append(page)
                slots = plan.token_slots[gi]
                if n_new == 1:
                    slots.append(table[start // ps] * ps + start % ps)
                else:
                    for p in range(start, total):
                        slots.append(table[p // ps] * ps + p % ps)
            req.length = total
        return plan

    # ------------------------------------------------------------------ views and checks

    def layer_kv(self, cache_layer: int) -> tuple[int, torch.Tensor, torch.Tensor]:
        """``(group index, keys, values)`` of a cache layer, each
        ``[pages, kv_heads, page_size, head_dim]``."""
        gi, li = self.layer_place[cache_layer]
        st = self.storage[gi]
        return gi, st[li, 0], st[li, 1]

    def layer_state(self, cache_layer: int) -> torch.Tensor | None:
        return self.state_arenas.get(cache_layer)

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def usage(self) -> float:
        """Fraction of all pages in use."""
        total = sum(p.num_pages for p in self.pools)
        free = sum(p.num_free for p in self.pools)
        return 0.0 if total == 0 else (total - free) / total

    def check(self) -> None:
        """Every page is free or held by exactly one request (raises ``CacheError``)."""
        for gi, pool in enumerate(self.pools):
            owner: dict[int, Hashable] = {}
            for req in self._requests.values():
                for page in req.tables[gi]:
                    if page < 0:
                        continue
                    if page in owner:
                        raise CacheError(f"group {gi}: page {page} held by {owner[page]!r} and {req.rid!r}")
                    owner[page] = req.rid
            free = pool.free_pages()
            if len(set(free)) != len(free):
                raise CacheError(f"group {gi}: a page is in the free list twice")
            if set(free) & set(owner):
                raise CacheError(f"group {gi}: a held page is in the free list")
            if len(free) + len(owner) != pool.num_pages:
                raise CacheError(
                    f"group {gi}: {pool.num_pages - len(free) - len(owner)} pages are lost"
                )
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("request slots are inconsistent")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a request slot is lost")
