"""A plain, slow implementation of the Llama decoder and of the sampler, for tests only.

Whole sequences, no cache, no batching, one function per part, written from the
reference's formulas (each function cites ``file:line`` of the reference project) and
sharing no code with the package under test.  Everything runs on the CPU in the dtype of
the tensors it is given (tests use float64 against the engine and float32 against the
golden outputs of the reference's own fp32 code, see ``tests/golden``).
"""

from __future__ import annotations

import math

import numpy as np
import torch


# ------------------------------------------------------------------------------- parts


def embed(table: torch.Tensor, ids) -> torch.Tensor:
    """``h0 = E[id]``, no scaling (models/llama/llama.py:159; distributed/embedding.py:102-105)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``w * x * rsqrt(mean(x^2) + eps)`` (models/blocks/rmsnorm.py:81-93)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(var + eps))


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """fp32 inverse frequencies with the optional llama3 rescale
    (models/blocks/rope.py:343-346 for the base table, :200-225 for the rescale)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    if scaling is None:
        return inv
    factor = scaling["factor"]
    low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
    L = scaling["original_max_position_embeddings"]
    out = inv.clone()
    for i in range(inv.numel()):
        f = inv[i]
        wavelen = 2 * math.pi / f
        scaled = f / factor if wavelen > L / low else f
        if not (wavelen < L / high) and not (wavelen > L / low):
            s = (L / wavelen - low) / (high - low)
            out[i] = (1 - s) * scaled / factor + s * scaled
        else:
            out[i] = scaled
    return out


def rope_cos_sin(positions, inv_freq: torch.Tensor, dtype: torch.dtype):
    """``ang = p * inv_freq`` in fp32, ``cat(ang, ang)``, cos/sin (models/blocks/rope.py:392-408).
    The angle product is taken in fp32 as the reference does; cos and sin are then
    evaluated in ``dtype`` (the reference rounds them to the model dtype)."""
    p = torch.as_tensor(positions, dtype=torch.float32)
    ang = (p[:, None] * inv_freq[None, :].float()).to(dtype)
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """``(-x_high, x_low)`` (models/blocks/rope.py:411-416)."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x * cos + rotate_half(x) * sin`` for ``x [T, heads, d]`` (models/blocks/rope.py:419-431)."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int | None = None, q_offset: int = 0) -> torch.Tensor:
    """``softmax(q k^T * scale + mask) v`` per head for ``q [Tq, nq, d]``, ``k, v [Tk, nkv, d]``;
    query ``i`` sits at position ``q_offset + i`` and sees keys ``<=`` its position (and
    ``> position - window`` with a window); query head ``h`` uses key/value head
    ``h // (nq / nkv)`` (cache/packed_attention.py:296-338)."""
    Tq, nq, d = q.shape
    Tk, nkv, _ = k.shape
    g = nq // nkv
    out = torch.empty_like(q)
    qpos = torch.arange(Tq) + q_offset
    kpos = torch.arange(Tk)
    invalid = kpos[None, :] > qpos[:, None]
    if window is not None:
        invalid = invalid | (kpos[None, :] < (qpos[:, None] - window + 1))
    for h in range(nq):
        kh = k[:, h // g, :]
        vh = v[:, h // g, :]
        scores = (q[:, h, :] @ kh.T) * scale
        scores = scores.masked_fill(invalid, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ vh
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """``down(silu(gate(x)) * up(x))`` (models/blocks/swiglu.py:45; models/blocks/activations.py:36-45)."""
    return (silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def attention_block(x, weights, prefix, cfg, cos, sin, window=None):
    """q/k/v projections, rope on q and k, causal GQA, output projection
    (models/blocks/gqa.py:111-155)."""
    T = x.shape[0]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = (x @ weights[prefix + "q_proj.weight"].T).view(T, nq, d)
    k = (x @ weights[prefix + "k_proj.weight"].T).view(T, nkv, d)
    v = (x @ weights[prefix + "v_proj.weight"].T).view(T, nkv, d)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, 1.0 / math.sqrt(d), window)
    return o.reshape(T, nq * d) @ weights[prefix + "o_proj.weight"].T


# ------------------------------------------------------------------------------- whole model


def normalise_config(raw: dict) -> dict:
    """The numbers the model needs from raw ``config.json`` keys (models/llama/llama.py:59-95)."""
    cfg = dict(raw)
    cfg.setdefault("num_key_value_heads", cfg["num_attention_heads"])
    if not cfg.get("head_dim"):
        cfg["head_dim"] = cfg["hidden_size"] // cfg["num_attention_heads"]
    rope = cfg.get("rope_parameters") or cfg.get("rope_scaling") or {}
    cfg["_theta"] = float(rope.get("rope_theta", cfg.get("rope_theta") or 10000.0))
    kind = rope.get("rope_type") or rope.get("type") or "default"
    cfg["_scaling"] = dict(rope) if kind == "llama3" else None
    return cfg


def llama_logits(weights: dict, raw_config: dict, ids, dtype=torch.float64) -> torch.Tensor:
    """Logits ``[T, vocab]`` of the whole sequence ``ids`` (models/llama/llama.py:159-172;
    residual structure models/blocks/transformer_block.py:107-153: ``h += attn(norm1(h))``,
    ``h += ffn(norm2(h))``, final norm, head; a tied head reuses the embedding table,
    models/llama/llama.py:143-147)."""
    cfg = normalise_config(raw_config)
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["rms_norm_eps"]
    inv_freq = rope_inv_freq(cfg["head_dim"], cfg["_theta"], cfg["_scaling"])
    cos, sin = rope_cos_sin(list(range(len(ids))), inv_freq, dtype)
    h = embed(w["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        a = rms_norm(h, w[p + "input_layernorm.weight"], eps)
        h = h + attention_block(a, w, p + "self_attn.", cfg, cos, sin)
        b = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + swiglu(b, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"])
    z = rms_norm(h, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return z @ head.T


def greedy_generate(weights: dict, raw_config: dict, prompt, n_new: int, dtype=torch.float64) -> list[int]:
    """Greedy continuation by re-running the whole sequence for every new token."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(torch.argmax(llama_logits(weights, raw_config, ids, dtype)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out


# ------------------------------------------------------------------------------- sampling


def philox_first_word(c0: int, c1: int, k0: int, k1: int) -> int:
    """Philox4x32-10 with counter ``(c0, c1, 0, 0)`` and key ``(k0, k1)``; first output word."""
    M0, M1 = 0xD2511F53, 0xCD9E8D57
    mask = 0xFFFFFFFF
    c2 = c3 = 0
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> 32, p0 & mask, p1 >> 32, p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        k0 = (k0 + 0x9E3779B9) & mask
        k1 = (k1 + 0xBB67AE85) & mask
    return c0


def gumbel_noise(vocab: int, seed: int, draw: int) -> np.ndarray:
    """``-log(-log(u_i))``, ``u_i = ((x_i >> 8) + 0.5) / 2^24`` in float64."""
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    u = np.array([((philox_first_word(i, draw, k0, k1) >> 8) + 0.5) / 16777216.0 for i in range(vocab)])
    return -np.log(-np.log(u))


def kept_mask(logits: np.ndarray, temperature: float, top_k: int, top_p: float) -> np.ndarray:
    """Which tokens survive top-k then top-p (engine/sampler.py:93-110): top-k keeps logits
    ``>=`` the k-th largest; top-p sorts descending, takes the cumulative softmax and drops
    a token when the mass *before* it already exceeds ``top_p`` (the boundary token stays)."""
    s = logits.astype(np.float64) / temperature
    keep = np.ones(s.shape, dtype=bool)
    if 0 < top_k < s.size:
        kth = np.sort(s)[::-1][top_k - 1]
        keep &= s >= kth
    if top_p < 1.0:
        masked = np.where(keep, s, -np.inf)
        order = np.argsort(-masked, kind="stable")
        e = np.exp(masked[order] - masked[order][0])
        probs = e / e.sum()
        before = np.concatenate([[0.0], np.cumsum(probs)[:-1]])
        drop = before > top_p
        keep2 = np.zeros_like(keep)
        keep2[order[~drop]] = True
        keep &= keep2
    return keep


def sample_reference(logits: np.ndarray, temperature: float, top_k: int, top_p: float, seed: int,
                     draw: int):
    """``(token, perturbed scores, kept mask)``: greedy at temperature 0, else the argmax of
    ``logit / T + Gumbel`` over the kept set (a draw from softmax over that set;
    engine/sampler.py:24-36,84-90 use an exponential race, the same distribution)."""
    if temperature == 0.0:
        return int(np.argmax(logits)), None, None
    keep = kept_mask(logits, temperature, top_k, top_p)
    score = logits.astype(np.float64) / temperature + gumbel_noise(logits.size, seed, draw)
    score = np.where(keep, score, -np.inf)
    return int(np.argmax(score)), score, keep
