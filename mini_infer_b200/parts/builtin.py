"""The parts that ship with the package: RMS norm, rotary position encoding, grouped-query
attention, SwiGLU feed-forward, token embedding, output head, the pre-norm arrangement.

Each class takes its sizes and constants from its ``PartSpec.params`` and its tensors from
``bind``.  The formulas follow the reference's blocks, cited per class.
"""

from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import (
    Arrangement,
    DeferredNorm,
    FeedForward,
    KVNeed,
    LayerCache,
    Mixer,
    Norm,
    ParamDecl,
    Part,
    PlanNeeds,
    Position,
    StepContext,
    StreamSink,
    register_arrangement,
    register_embedding,
    register_feed_forward,
    register_head,
    register_mixer,
    register_norm,
    register_position,
)


def _as_compute(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A matrix operand in the compute dtype (a no-op when it is stored that way)."""
    return t if t.dtype == dtype else t.to(dtype)


class Linear:
    """``y = x W^T`` with ``W [out, in]`` kept in the compute dtype.

    ``x`` may be a ``DeferredNorm`` whose statistics are row sums of squares (the product then
    finishes the norm in its epilogue), and ``into_stream`` adds the product to a sink's stream;
    ``fusable`` says whether this matrix and row count have those forms."""

    def __init__(self, weight: torch.Tensor) -> None:
        if weight.dim() != 2 or not weight.is_contiguous():
            raise ValueError("Linear needs a contiguous [out, in] matrix")
        self.weight = weight

    def __call__(self, x, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        if isinstance(x, DeferredNorm):
            if x.kind != "rms":
                raise ValueError(f"this product cannot finish a norm of kind {x.kind!r}")
            return ops.linear(x.x, self.weight, out_dtype, row_stats=x.stats)
        return ops.linear(x, self.weight, out_dtype)

    def fusable(self, n_rows: int, kind: str = "rms") -> bool:
        return kind == "rms" and ops.linear_fusable(n_rows, self.weight)

    def into_stream(self, x: torch.Tensor, sink: StreamSink) -> DeferredNorm:
        if sink.kind != "rms":
            raise ValueError(f"this product cannot finish a norm of kind {sink.kind!r}")
        gain, eps = sink.payload
        y, stats = ops.linear_into_stream(x, self.weight, sink.residual, gain, eps)
        return DeferredNorm(sink.norm, sink.kind, y, stats, sink.residual)


# ----------------------------------------------------------------------------- norm


class RMSNorm(Norm):
    """``w * r * rsqrt(mean(r^2) + eps)`` with ``r = x + residual`` in fp32
    (reference ``models/blocks/rmsnorm.py:63-93``; the residual sum is kept in fp32 here
    instead of being rounded to the model dtype).

    params: ``hidden_size``, ``eps``.  tensors: ``weight [hidden_size]``.
    """

    deferred_kind = "rms"

    def param_decls(self):
        return {"weight": ParamDecl((int(self.param("hidden_size")),), "gain")}

    def bind(self, tensors, dtype, device):
        w = tensors["weight"]
        # a gain stored in 32-bit stays 32-bit; anything else follows the compute dtype
        self.weight = w if w.dtype == torch.float32 else w.to(dtype)
        self.eps = float(self.param("eps"))

    def stream_sink(self, residual, n_rows):
        if (not ops.fused_norms_enabled() or residual is None
                or n_rows > ops.TMA_GEMM_FUSED_ROWS or not residual.is_cuda):
            return None
        if getattr(self, "_gain32", None) is None:
            self._gain32 = self.weight.to(torch.float32).contiguous()   # the products' epilogues read fp32
        return StreamSink(self, self.deferred_kind, residual, (self._gain32, self.eps))

    def forward(self, x, residual, rows=None):
        if isinstance(x, DeferredNorm):
            if x.norm is not self or rows is not None:
                raise ValueError("a deferred norm was handed to another norm than the one it was made for")
            return x, x.residual
        if rows is not None:
            return ops.add_rmsnorm(x, self.weight, self.eps, residual_in=residual, rows=rows), None
        new_residual = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        out = ops.add_rmsnorm(x, self.weight, self.eps, residual_in=residual,
                              residual_out=new_residual)
        return out, new_residual


# ----------------------------------------------------------------------------- position


def rotary_inv_freq(head_dim: int, theta: float, rotary_dim: int | None = None,
                    scaling: dict | None = None) -> torch.Tensor:
    """fp32 rotation frequencies ``theta^(-2i/d)``, optionally with the llama3 rescale.

    The rescale sorts frequencies by wavelength into three bands: short waves (below
    ``L / high_freq_factor``, ``L`` the original context length) are kept, long waves (above
    ``L / low_freq_factor``) are slowed down by ``factor``, and the band between is a blend of
    both that is linear in ``L / wavelength``.  Every intermediate is fp32 and the
    operations run in the order of the reference's ``models/blocks/rope.py:200-225``, so
    the table comes out bit-equal to the reference's (a test compares them).
    """
    width = head_dim if rotary_dim is None else rotary_dim
    exponent = torch.arange(0, width, 2, dtype=torch.float32) / head_dim
    freq = 1.0 / (theta ** exponent)
    if scaling is None:
        return freq
    slow_down = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    context = int(scaling["original_max_position_embeddings"])
    wave = 2 * math.pi / freq
    is_long, is_short = wave > context / low, wave < context / high
    slowed = torch.where(is_long, freq / slow_down, freq)
    blend = (context / wave - low) / (high - low)          # 0 at the long edge, 1 at the short edge
    blended = (1 - blend) * slowed / slow_down + blend * slowed
    in_between = ~is_short * ~is_long
    return torch.where(in_between, blended, slowed)


class RotaryPosition(Position):
    """Rotary encoding, half layout: dim ``j`` pairs with ``j + rotary_dim/2``
    (reference ``models/blocks/rope.py:392-431``).  Angles ``p * inv_freq`` and their sine
    and cosine are fp32 and computed in the kernel; each rotated value is rounded once.

    params: ``head_dim``, ``theta``, optional ``rotary_dim`` (default ``head_dim``),
    optional ``scaling`` (the llama3 mapping).
    """

    def bind(self, tensors, dtype, device):
        d = int(self.param("head_dim"))
        self.rotary_dim = int(self.spec.params.get("rotary_dim") or d)
        self.inv_freq = rotary_inv_freq(
            d, float(self.param("theta")), self.rotary_dim, self.spec.params.get("scaling")
        ).to(device)
        # layers with the same frequencies share one table per step
        self._table_key = (d, self.rotary_dim, float(self.param("theta")), repr(self.spec.params.get("scaling")))

    def encode(self, qkv, nq, nkv, head_dim, ctx):
        ops.rope_write(qkv, nq, nkv, head_dim, positions=ctx.positions, inv_freq=self.inv_freq,
                       rotary_dim=self.rotary_dim)

    def step_table(self, ctx, head_dim):
        """Sines and cosines of this step's positions for a mixer that rotates by itself, or
        None where that is not possible (a rotary width below the head size).  Layers share one
        table per step: it depends on the positions and the frequencies only."""
        if self.rotary_dim != head_dim:
            return None
        key = ("rope_table", self._table_key)
        table = ctx.scratch.get(key)
        if table is None:
            table = ctx.scratch[key] = ops.rope_table(ctx.positions, self.inv_freq)
        return table

    def rotate_and_store(self, qkv, nq, nkv, head_dim, ctx, cache):
        if cache.writes and cache.k is not None:
            ops.rope_write(qkv, nq, nkv, head_dim, positions=ctx.positions,
                           inv_freq=self.inv_freq, rotary_dim=self.rotary_dim,
                           slots=ctx.groups[cache.group].slots, kcache=cache.k, vcache=cache.v)
        else:
            self.encode(qkv, nq, nkv, head_dim, ctx)


# ----------------------------------------------------------------------------- mixer


class GroupedQueryAttention(Mixer):
    """Causal attention with ``num_heads`` query heads sharing ``num_kv_heads`` key/value
    heads over the paged cache (reference ``models/blocks/gqa.py:111-155`` and
    ``cache/packed_attention.py:242-340``): one merged q/k/v projection, position encoding
    of q and k, k/v written to pages, softmax(q k^T * scale + causal [+ window]) v in fp32,
    output projection.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``; optional
    ``window`` (keys older than ``window - 1`` positions are not seen), ``scale``
    (default ``head_dim ** -0.5``).
    tensors: ``q_proj.weight``, ``k_proj.weight``, ``v_proj.weight``, ``o_proj.weight``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.nq = int(self.param("num_heads"))
        self.nkv = int(self.param("num_kv_heads"))
        self.d = int(self.param("head_dim"))
        w = self.spec.params.get("window")
        self.window = int(w) if w else None
        s = self.spec.params.get("scale")
        self.scale = float(s) if s else self.d ** -0.5
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads cannot share {self.nkv} key/value heads")
        if self.d % 16 or not 16 <= self.d <= 256:
            raise ValueError(f"head_dim {self.d} is not a multiple of 16 in [16, 256]")

    def param_decls(self):
        H, nq, nkv, d = self.hidden, self.nq, self.nkv, self.d
        return {
            "q_proj.weight": ParamDecl((nq * d, H)),
            "k_proj.weight": ParamDecl((nkv * d, H)),
            "v_proj.weight": ParamDecl((nkv * d, H)),
            "o_proj.weight": ParamDecl((H, nq * d)),
        }

    def cache_need(self):
        return KVNeed(self.nkv, self.d, self.window)

    def plan_needs(self):
        return PlanNeeds(ops.attention_tile_sizes(self.nq // self.nkv))

    def bind(self, tensors, dtype, device):
        qkv = torch.cat(
            [_as_compute(tensors[n], dtype) for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")],
            dim=0,
        ).contiguous()
        self.qkv_proj = Linear(qkv)
        self.o_proj = Linear(_as_compute(tensors["o_proj.weight"], dtype).contiguous())

    def takes_deferred_norm(self, n_rows, kind):
        return self.qkv_proj.fusable(n_rows, kind)

    def adds_to_stream(self, n_rows, kind):
        return self.o_proj.fusable(n_rows, kind)

    def forward(self, x, ctx: StepContext, cache: LayerCache, position, into=None):
        nq, nkv, d = self.nq, self.nkv, self.d
        qkv = self.qkv_proj(x)
        table = None
        if (position is not None and cache.k is not None
                and ops.decode_rope_fusable(x.dtype, d, ctx.decode_only, ctx.n_requests)):
            table = position.step_table(ctx, d)   # the decode kernel rotates q and stores the new k, v itself
        if table is not None:
            pass
        elif position is not None:
            position.rotate_and_store(qkv, nq, nkv, d, ctx, cache)
        elif cache.writes:
            ops.rope_write(qkv, nq, nkv, d, slots=ctx.groups[cache.group].slots,
                           kcache=cache.k, vcache=cache.v)
        out = torch.empty((ctx.n_tokens, nq * d), dtype=x.dtype, device=x.device)
        ops.attention(qkv, qkv.stride(0), out, cache, ctx, nq, nkv, d, self.scale, self.window or 0,
                      rope_table=table)
        return self.o_proj(out) if into is None else self.o_proj.into_stream(out, into)


# ----------------------------------------------------------------------------- feed-forward


class SwiGLU(FeedForward):
    """``down(silu(gate(x)) * up(x))``, no biases (reference ``models/blocks/swiglu.py:35-46``,
    ``models/blocks/activations.py:36-45``).  gate and up are one merged product whose rows
    alternate (gate 0, up 0, gate 1, up 1, ...), so that the activation can run in the
    product's epilogue, where both halves of a pair sit side by side; SiLU and the product
    are fp32 per element.

    params: ``hidden_size``, ``intermediate_size``.
    tensors: ``gate_proj.weight``, ``up_proj.weight``, ``down_proj.weight``.
    """

    def param_decls(self):
        H, I = int(self.param("hidden_size")), int(self.param("intermediate_size"))
        return {
            "gate_proj.weight": ParamDecl((I, H)),
            "up_proj.weight": ParamDecl((I, H)),
            "down_proj.weight": ParamDecl((H, I)),
        }

    def bind(self, tensors, dtype, device):
        gate, up = _as_compute(tensors["gate_proj.weight"], dtype), _as_compute(tensors["up_proj.weight"], dtype)
        gate_up = torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()
        self.gate_up_proj = Linear(gate_up)
        self.down_proj = Linear(_as_compute(tensors["down_proj.weight"], dtype).contiguous())

    def takes_deferred_norm(self, n_rows, kind):
        return self.gate_up_proj.fusable(n_rows, kind)

    def adds_to_stream(self, n_rows, kind):
        return self.down_proj.fusable(n_rows, kind)

    def forward(self, x, ctx, into=None):
        if isinstance(x, DeferredNorm):
            if x.kind != "rms":
                raise ValueError(f"this product cannot finish a norm of kind {x.kind!r}")
            h = ops.linear_swiglu(x.x, self.gate_up_proj.weight, row_stats=x.stats)
        else:
            h = ops.linear_swiglu(x, self.gate_up_proj.weight)
        return self.down_proj(h) if into is None else self.down_proj.into_stream(h, into)


# ----------------------------------------------------------------------------- embedding / head


class TokenEmbedding(Part):
    """``h0 = E[token]``, no scale (reference ``models/llama/llama.py:104,159``).

    params: ``vocab_size``, ``hidden_size``.  tensors: ``weight [vocab, hidden]``.
    """

    def param_decls(self):
        return {"weight": ParamDecl((int(self.param("vocab_size")), int(self.param("hidden_size"))))}

    def bind(self, tensors, dtype, device):
        self.weight = _as_compute(tensors["weight"], dtype).contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        return ops.embedding(self.weight, ctx.token_ids)


class OutputHead(Part):
    """``logits = z W^T`` in fp32 (reference ``models/llama/llama.py:169-172``).  With
    ``tied`` the embedding's table is the weight and no tensor of its own is expected.

    params: ``vocab_size``, ``hidden_size``, ``tied``.  tensors: ``weight`` unless tied.
    """

    @property
    def tied(self) -> bool:
        return bool(self.spec.params.get("tied", False))

    def param_decls(self):
        if self.tied:
            return {}
        return {"weight": ParamDecl((int(self.param("vocab_size")), int(self.param("hidden_size"))))}

    def bind(self, tensors, dtype, device, tied_weight: torch.Tensor | None = None):
        if self.tied:
            if tied_weight is None:
                raise ValueError("a tied head needs the embedding's table")
            self.proj = Linear(tied_weight)
        else:
            self.proj = Linear(_as_compute(tensors["weight"], dtype).contiguous())

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        return self.proj(z, out_dtype=torch.float32)


# ----------------------------------------------------------------------------- arrangement


class PreNormBlock(Arrangement):
    """``h += mixer(norm1(h)); h += ffn(norm2(h))`` with every addition folded into the
    following norm (reference ``models/blocks/transformer_block.py:107-120,140-153``): the
    block receives the previous branch output ``x`` and the fp32 stream ``residual``, and
    returns its feed-forward output with the stream that does not yet include it.

    Where the parts on both sides of a norm say they can (few rows, bfloat16), the branch's last
    product adds its result to the stream itself and the product after the norm finishes the
    norm in its epilogue, so that the norm launches nothing: within the block for the second
    norm, and across blocks when the layer that follows gave its ``entry``.
    """

    def entry(self):
        return self.mixer_norm, self.mixer

    @staticmethod
    def _sink(producer, norm, consumer, residual, n_rows):
        kind = norm.deferred_kind
        if (kind is None or residual is None or not producer.adds_to_stream(n_rows, kind)
                or not consumer.takes_deferred_norm(n_rows, kind)):
            return None
        return norm.stream_sink(residual, n_rows)

    def forward(self, x, residual, ctx, cache, following=None):
        n = ctx.n_tokens
        a, residual = self.mixer_norm.forward(x, residual)
        sink = self._sink(self.mixer, self.feed_forward_norm, self.feed_forward, residual, n)
        if sink is None:
            h = self.mixer.forward(a, ctx, cache, self.position)
        else:
            h = self.mixer.forward(a, ctx, cache, self.position, into=sink)
        b, residual = self.feed_forward_norm.forward(h, residual)
        sink = self._sink(self.feed_forward, following[0], following[1], residual, n) if following else None
        if sink is None:
            f = self.feed_forward.forward(b, ctx)
        else:
            f = self.feed_forward.forward(b, ctx, into=sink)
        return f, residual


register_norm("rmsnorm", RMSNorm, replace=True)
register_position("rotary", RotaryPosition, replace=True)
register_mixer("gqa_attention", GroupedQueryAttention, replace=True)
register_feed_forward("swiglu", SwiGLU, replace=True)
register_embedding("token_embedding", TokenEmbedding, replace=True)
register_head("linear_head", OutputHead, replace=True)
register_arrangement("prenorm", PreNormBlock, replace=True)
