"""The plain implementation against the reference project's own fp32 outputs (golden
files made by tests/golden/make_golden.py) and against itself, part by part."""

import hashlib
import math
import os

import numpy as np
import pytest
import torch

import plain_impl as P
from tiny_configs import TINY, load_state

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _checksum(state):
    h = hashlib.sha256()
    for name in sorted(state):
        h.update(name.encode())
        h.update(state[name].float().numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_plain_matches_reference_golden(which, model_dirs):
    gold = np.load(os.path.join(GOLDEN, f"tiny_{which}.npz"))
    state = load_state(model_dirs[which])
    assert _checksum(state) == str(gold["weights_sha256"]), "seeded random weights changed"
    ids = gold["prompt"].tolist()
    logits32 = P.llama_logits(state, TINY[which], ids, dtype=torch.float32).numpy()
    logits64 = P.llama_logits(state, TINY[which], ids, dtype=torch.float64).numpy()
    scale = np.abs(gold["logits"]).max()
    assert np.abs(logits32 - gold["logits"]).max() <= 2e-5 * max(1.0, scale)
    # the golden logits carry the fp32 rounding of the reference's own run (a few 1e-5 with
    # peaked attention); the float64 run of the same formulas must agree to that level
    assert np.abs(logits64 - gold["logits"]).max() <= 1e-4 * max(1.0, scale)


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_inv_freq_bit_equal_to_reference(which):
    """Both the plain implementation's table and the product's own (the one the rotary kernel
    is given) equal the reference's fp32 table bit for bit."""
    from mini_infer_b200.config import load_config
    from mini_infer_b200.parts.builtin import rotary_inv_freq

    gold = np.load(os.path.join(GOLDEN, f"tiny_{which}.npz"))
    cfg = P.normalise_config(TINY[which])
    mine = P.rope_inv_freq(cfg["head_dim"], cfg["_theta"], cfg["_scaling"]).numpy()
    assert np.array_equal(mine, gold["inv_freq"])
    arch, typed = load_config(TINY[which])
    position = arch.assemble(typed).layers[0].position
    product = rotary_inv_freq(position.params["head_dim"], position.params["theta"],
                              position.params.get("rotary_dim"), position.params.get("scaling"))
    assert product.dtype == torch.float32
    assert np.array_equal(product.numpy(), gold["inv_freq"])


def test_inv_freq_check_values():
    """Configuration A's table (theta 1e4, head size 16, llama3 factor 8, low 1, high 4, original
    length 64): one frequency kept, two blended, five divided by 8."""
    from mini_infer_b200.parts.builtin import rotary_inv_freq

    cfg = P.normalise_config(TINY["A"])
    want = [1.0, 2.4438e-01, 1.3042e-02, 3.9528e-03, 1.2500e-03, 3.9528e-04, 1.2500e-04, 3.9528e-05]
    for table in (P.rope_inv_freq(16, 10000.0, cfg["_scaling"]), rotary_inv_freq(16, 10000.0, None, cfg["_scaling"])):
        assert np.allclose(table.numpy(), want, rtol=1e-4)


def test_llama3_rescale_has_three_bands():
    cfg = P.normalise_config(TINY["A"])
    plain = P.rope_inv_freq(16, 10000.0, None)
    scaled = P.rope_inv_freq(16, 10000.0, cfg["_scaling"])
    ratio = (scaled / plain).tolist()
    assert ratio[0] == 1.0                       # short wavelength: kept
    assert all(abs(r - 1 / 8) < 1e-6 for r in ratio[3:])  # long: divided by the factor
    assert 1 / 8 < ratio[1] < 1.0 and 1 / 8 < ratio[2] < 1.0  # blended


def test_attention_is_causal_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8, dtype=torch.float64), torch.randn(6, 2, 8, dtype=torch.float64), torch.randn(6, 2, 8, dtype=torch.float64)
    full = P.causal_attention(q, k, v, 0.5)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0           # the future must not matter
    assert torch.allclose(P.causal_attention(q, k2, v2, 0.5)[:4], full[:4])
    assert torch.allclose(full[0], v[0].repeat_interleave(2, dim=0))  # first query sees key 0 only
    win = P.causal_attention(q, k, v, 0.5, window=1)
    assert torch.allclose(win, v.repeat_interleave(2, dim=1))         # window 1: own value
    # a portion at an offset equals the tail of the whole
    tail = P.causal_attention(q[3:], k, v, 0.5, q_offset=3)
    assert torch.allclose(tail, full[3:])


def test_rope_is_a_rotation_by_relative_position():
    inv = P.rope_inv_freq(8, 10000.0, None)
    cos, sin = P.rope_cos_sin([3, 10], inv, torch.float64)
    x = torch.randn(2, 1, 8, dtype=torch.float64)
    y = P.apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # <rope(a, p), rope(b, q)> depends on p - q only
    a, b = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    def dot(p, q):
        cp, sp = P.rope_cos_sin([p], inv, torch.float64)
        cq, sq = P.rope_cos_sin([q], inv, torch.float64)
        return float((P.apply_rope(a, cp, sp) * P.apply_rope(b, cq, sq)).sum())
    assert math.isclose(dot(5, 2), dot(13, 10), rel_tol=1e-9)


def test_rms_norm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    out = P.rms_norm(x, w, 0.0)
    assert torch.allclose(out, torch.tensor([[2 * 3 / math.sqrt(12.5), 0.5 * 4 / math.sqrt(12.5)]], dtype=torch.float64))
    eye = torch.eye(2, dtype=torch.float64)
    y = P.swiglu(x, eye, eye, eye)
    assert torch.allclose(y, x * x / (1 + torch.exp(-x)))


def test_sampler_reference():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=50).astype(np.float32)
    assert P.sample_reference(logits, 0.0, 0, 1.0, 1, 0)[0] == int(np.argmax(logits))
    keep = P.kept_mask(logits, 1.0, 5, 1.0)
    assert keep.sum() == 5 and keep[np.argsort(-logits)[:5]].all()
    keep = P.kept_mask(logits, 1.0, 0, 1e-6)
    assert keep.sum() == 1 and keep[np.argmax(logits)]
    # draws follow softmax
    counts = np.zeros(50)
    small = logits[:8]
    for d in range(4000):
        counts[P.sample_reference(small, 0.7, 0, 1.0, 1234, d)[0]] += 1
    probs = np.exp(small / 0.7) / np.exp(small / 0.7).sum()
    assert np.abs(counts[:8] / 4000 - probs).max() < 0.03
    # same seed and draw index: same token; the noise does not depend on anything else
    assert P.sample_reference(small, 0.7, 0, 1.0, 99, 3)[0] == P.sample_reference(small, 0.7, 0, 1.0, 99, 3)[0]
