"""Interfaces of the parts a decoder is put together from, and their registries.

A *part* is built from a :class:`~.spec.PartSpec` alone (its sizes and constants); it
declares the tensors it needs under local names, receives them in ``bind`` and does its
work in ``forward``.  Four families exist, each with a registry keyed by ``kind``:

``Mixer``         mixes information across the tokens of a request (attention here).
                  Declares what it keeps between steps: per-token keys/values in pages
                  (``cache_need``) and/or a fixed-size per-request state (``state_need``).
``FeedForward``   per-token transformation (dense SwiGLU here; routed experts fit the
                  same interface).
``Norm``          ``forward(x, residual) -> (normed, new_residual)``; the residual stream
                  is fp32.
``Position``      how positions enter a mixer's queries and keys.

An *arrangement* says where the norms and the residual additions of a layer stand.

No part knows which model it is in: everything it needs is in its spec, in the tensors it
is bound to, and in the :class:`StepContext` of the step.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, ClassVar

import torch

from .spec import PartSpec


# ----------------------------------------------------------------------------- declarations


@dataclass(frozen=True)
class ParamDecl:
    """A tensor a part needs.  ``role`` guides random initialisation and dtype policy:

    ``matrix``  operand of a matrix product; converted to the compute dtype when bound
    ``gain``    multiplicative vector of a norm; a 32-bit stored gain stays 32-bit
    ``table``   anything else (kept as loaded)
    """

    shape: tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class KVNeed:
    """Per-token keys and values kept in pages: ``kv_heads * head_dim`` numbers each per
    token.  ``window``: only the last ``window`` positions are ever read (None: all)."""

    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """A per-request state of fixed size (zeroed when a request is admitted)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class PlanNeeds:
    """What a mixer wants the step planner to prepare each step.

    ``q_tile_tokens``: for each value n, a list of tiles of at most n consecutive query
    tokens of one request (``StepContext.q_tiles(n)``).
    """

    q_tile_tokens: frozenset[int] = frozenset()


# ----------------------------------------------------------------------------- step context


@dataclass
class GroupView:
    """One cache group as a step sees it (device tensors are int32)."""

    page_size: int
    window: int | None
    block_table: torch.Tensor          # [request slots, max_pages] page ids of this group, resident on the device
    slots: torch.Tensor                # [tokens] flat slot (page * page_size + offset) per new token
    table_rows: torch.Tensor | None = None   # [requests] row of block_table of each request (None: its index)


@dataclass
class LayerCache:
    """What one schedule entry's mixer gets from the cache manager."""

    group: int | None = None           # index into StepContext.groups
    k: torch.Tensor | None = None      # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor | None = None
    state: torch.Tensor | None = None  # [request slots, *StateNeed.shape]
    writes: bool = True


@dataclass
class StepContext:
    """Everything a part may know about the batch of one step.

    Host lists and their device copies describe the same thing; kernels read the device
    tensors, Python code that must loop over requests (a toy mixer) reads the lists.
    """

    dtype: torch.dtype
    device: torch.device
    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor            # [tokens] int32
    positions: torch.Tensor            # [tokens] int32 absolute position of each token
    q_start: torch.Tensor              # [requests] int32 first row of each request's portion
    q_len: torch.Tensor                # [requests] int32
    kv_len: torch.Tensor               # [requests] int32 tokens held after this step
    state_slot: torch.Tensor           # [requests] int32 row of each request in state arenas
    host_q_start: list[int] = field(default_factory=list)
    host_q_len: list[int] = field(default_factory=list)
    host_kv_len: list[int] = field(default_factory=list)
    host_state_slot: list[int] = field(default_factory=list)
    groups: list[GroupView] = field(default_factory=list)
    tiles: dict[int, tuple[torch.Tensor, torch.Tensor, int]] = field(default_factory=dict)
    decode_only: bool = False          # every request brings exactly one token
    # a mixed step: the requests that bring one token (their rows of q, their lengths, their rows
    # of the block tables) and the query tiles of the other requests alone
    n_single: int = 0
    single_q_start: torch.Tensor | None = None
    single_kv_len: torch.Tensor | None = None
    single_rows: torch.Tensor | None = None
    tiles_multi: dict[int, tuple[torch.Tensor, torch.Tensor, int]] = field(default_factory=dict)
    max_kv_len: int = 0
    # per cache group: (triples, count, capacity) of the page ids the step scatters into the
    # block tables before its first kernel (the step runner's business, not a part's)
    table_updates: list = field(default_factory=list)
    # what parts of different layers share within one step (a table that depends on the step's
    # positions only, say): filled by whoever needs it first
    scratch: dict = field(default_factory=dict)

    def q_tiles(self, tokens: int) -> tuple[torch.Tensor, torch.Tensor, int]:
        """``(tile_request, tile_first_token, n_tiles)`` for tiles of ``tokens`` tokens."""
        try:
            return self.tiles[tokens]
        except KeyError:
            raise KeyError(
                f"no query tiles of {tokens} tokens were planned; a mixer must announce "
                "the tile sizes it uses in plan_needs()"
            ) from None


# ----------------------------------------------------------------------------- part families


class Part:
    kind: ClassVar[str] = ""
    # A captured step replays the device work of ``forward`` without running its Python again.
    # A part whose ``forward`` reads the host lists of the StepContext, synchronises with the
    # device or changes Python state sets this to False; steps of its model then always run
    # kernel by kernel.
    graph_safe: ClassVar[bool] = True

    def __init__(self, spec: PartSpec) -> None:
        self.spec = spec

    def param_decls(self) -> dict[str, ParamDecl]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        """Receive the declared tensors (already on ``device``); ``dtype`` is the compute
        dtype of activations (float32 or bfloat16)."""

    def param(self, name: str, default: Any = None) -> Any:
        if name in self.spec.params:
            return self.spec.params[name]
        if default is not None:
            return default
        raise KeyError(f"part {self.spec.kind!r} needs parameter {name!r}")


class Position(Part):
    """Position encoding applied to the queries and keys of a mixer.

    ``rotate_and_store`` receives the packed projection ``qkv [tokens, (nq + 2 nkv) * d]``
    and must leave encoded queries and keys in it and, when ``cache.writes``, store the
    encoded keys and the values at ``ctx.groups[cache.group].slots``.  The default does
    the two halves separately through ``encode`` and the store kernel; a part with a
    fused kernel overrides ``rotate_and_store``.
    """

    def encode(self, qkv: torch.Tensor, nq: int, nkv: int, head_dim: int, ctx: StepContext) -> None:
        raise NotImplementedError

    def step_table(self, ctx: StepContext, head_dim: int) -> torch.Tensor | None:
        """For an encoding that is a rotation of the half layout (dim ``j`` with ``j + head_dim /
        2``): fp32 ``[tokens, head_dim]``, per token the sines then the cosines of its angles, so
        that a mixer whose kernel rotates by itself can skip ``rotate_and_store``.  None (the
        default): the encoding goes through ``rotate_and_store``."""
        return None

    def rotate_and_store(self, qkv: torch.Tensor, nq: int, nkv: int, head_dim: int,
                         ctx: StepContext, cache: LayerCache) -> None:
        from ..csrc import ops

        self.encode(qkv, nq, nkv, head_dim, ctx)
        if cache.writes and cache.k is not None:
            ops.rope_write(qkv, nq, nkv, head_dim, slots=ctx.groups[cache.group].slots,
                           kcache=cache.k, vcache=cache.v)


class StreamSink:
    """Where a branch's last product may put its result instead of returning it: added to the
    fp32 ``residual`` stream in place, with what ``norm`` (the norm that follows) needs to do the
    rest without a kernel of its own.  Made by ``Norm.stream_sink``; ``kind`` is the norm's
    ``deferred_kind`` and says what ``payload`` holds (``"rms"``: the gain in fp32 and eps)."""

    __slots__ = ("norm", "kind", "residual", "payload")

    def __init__(self, norm: "Norm", kind: str, residual: torch.Tensor, payload: Any) -> None:
        self.norm, self.kind, self.residual, self.payload = norm, kind, residual, payload


class DeferredNorm:
    """A norm's input whose addition to the stream has happened and whose normalisation is left
    to the product that reads it: ``x`` (the stream times the norm's gain, in the compute dtype),
    ``stats`` (what that product needs to finish the norm; for kind ``"rms"`` the sums of squares
    per row) and the updated ``residual`` stream.  The norm it was made for hands it on untouched;
    a part takes it only if it said so (``takes_deferred_norm``)."""

    __slots__ = ("norm", "kind", "x", "stats", "residual")

    def __init__(self, norm: "Norm", kind: str, x: torch.Tensor, stats: Any, residual: torch.Tensor) -> None:
        self.norm, self.kind, self.x, self.stats, self.residual = norm, kind, x, stats, residual

    @property
    def dtype(self) -> torch.dtype:
        return self.x.dtype

    @property
    def device(self) -> torch.device:
        return self.x.device

    @property
    def shape(self) -> torch.Size:
        return self.x.shape


class Norm(Part):
    # What kind of unfinished norm this class can leave to the products around it (``"rms"``: the
    # product before adds to the stream, multiplies by the gain and leaves sums of squares; the
    # product after divides by the root mean square), or None: the norm always runs by itself.
    deferred_kind: ClassVar[str | None] = None

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None,
                rows: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:
        """``(normed, new_residual)``; ``residual`` is the fp32 stream or None (first norm).

        With ``rows`` (int32 indices) only those rows are normalised and no residual is
        returned.  A norm that hands out sinks (below) is given back what was made from them, a
        ``DeferredNorm``, as ``x``, and returns it with its residual, launching nothing."""
        raise NotImplementedError

    def stream_sink(self, residual: torch.Tensor, n_rows: int) -> StreamSink | None:
        """A sink for the branch before this norm, or None when this norm (or this step: its
        dtype, its number of rows) has no fused form; the branch then returns its output and
        ``forward`` adds and normalises as usual."""
        return None


class Mixer(Part):
    def cache_need(self) -> KVNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def plan_needs(self) -> PlanNeeds:
        return PlanNeeds()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache,
                position: Position | None) -> torch.Tensor:
        raise NotImplementedError

    # Optional, for arrangements that let additions and norms ride on a branch's products.  A
    # part that answers True to the first is called with ``x`` a ``DeferredNorm`` of that kind;
    # one that answers True to the second is called with ``into=sink`` (a sink of that kind) and
    # returns a ``DeferredNorm``.  Parts that know nothing of this inherit False and are called
    # as above.
    def takes_deferred_norm(self, n_rows: int, kind: str) -> bool:
        return False

    def adds_to_stream(self, n_rows: int, kind: str) -> bool:
        return False


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def takes_deferred_norm(self, n_rows: int, kind: str) -> bool:
        return False

    def adds_to_stream(self, n_rows: int, kind: str) -> bool:
        return False


class Arrangement:
    """A layer: a mixer and a feed-forward behind their norms.

    ``forward(x, residual, ctx, cache) -> (x, residual)`` where ``x`` is the last branch
    output not yet added to the fp32 ``residual`` stream (``residual`` is None before the
    first layer, when ``x`` is the embedding).
    """

    kind: ClassVar[str] = ""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm, position: Position | None) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.position = position

    def parts(self) -> list[Part]:
        ps: list[Part] = [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]
        if self.position is not None:
            ps.append(self.position)
        return ps

    def forward(self, x, residual, ctx: StepContext, cache: LayerCache):
        raise NotImplementedError

    def entry(self) -> tuple[Norm, Part] | None:
        """The norm a layer begins with and the part that reads it, for the layer before (which
        may then add its last branch to the stream itself and leave the norm to that part,
        ``forward(..., following=entry)``), or None: the layer wants a plain ``(x, residual)``.
        An arrangement that returns an entry also takes the ``following`` argument."""
        return None


# ----------------------------------------------------------------------------- registries

_REGISTRIES: dict[str, dict[str, Callable[..., Any]]] = {
    "mixer": {},
    "feed_forward": {},
    "norm": {},
    "position": {},
    "arrangement": {},
    "embedding": {},
    "head": {},
}


def _register(family: str, kind: str, cls, replace: bool) -> None:
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise ValueError(f"{family} kind {kind!r} is already registered")
    reg[kind] = cls


def register_mixer(kind: str, cls, *, replace: bool = False) -> None:
    _register("mixer", kind, cls, replace)


def register_feed_forward(kind: str, cls, *, replace: bool = False) -> None:
    _register("feed_forward", kind, cls, replace)


def register_norm(kind: str, cls, *, replace: bool = False) -> None:
    _register("norm", kind, cls, replace)


def register_position(kind: str, cls, *, replace: bool = False) -> None:
    _register("position", kind, cls, replace)


def register_arrangement(kind: str, cls, *, replace: bool = False) -> None:
    _register("arrangement", kind, cls, replace)


def register_embedding(kind: str, cls, *, replace: bool = False) -> None:
    _register("embedding", kind, cls, replace)


def register_head(kind: str, cls, *, replace: bool = False) -> None:
    _register("head", kind, cls, replace)


def lookup(family: str, kind: str):
    from . import builtin  # noqa: F401  (registers the parts that ship with the package)

    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        raise ValueError(
            f"unknown {family} kind {kind!r}; registered: {sorted(_REGISTRIES[family])}"
        ) from None


def build_part(family: str, spec: PartSpec):
    return lookup(family, spec.kind)(spec)
