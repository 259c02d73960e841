"""How a decode step's keys are cut into slices (``ops.decode_plan``): pure arithmetic, no GPU."""

from __future__ import annotations

import random

from mini_infer_b200.csrc import ops

SMS = 148


def _chunks(kl: int, window: int) -> int:
    lo = max(0, kl - window) if window else 0
    return max(1, -(-kl // 64) - lo // 64)


def test_equal_lengths_give_the_uniform_rule():
    """Requests of one length: as many slices as fill about two blocks per SM, at least four
    chunks each."""
    for batch, kv, nq, nkv, want in [(8, 2049, 32, 8, 4), (1, 2049, 32, 8, 8), (64, 2049, 32, 8, 1),
                                     (1, 100, 32, 8, 1), (2, 40000, 32, 8, 16), (8, 2049, 64, 8, 4)]:
        n, per = ops.decode_plan([kv] * batch, 0, ops.decode_blocks_per_request(nq, nkv), SMS)
        assert n == want, (batch, kv, n)
        assert n * per >= _chunks(kv, 0)
        assert n == 1 or per >= 4


def test_one_long_request_is_cut_and_the_short_ones_stay_whole():
    lens = [30000] + [1500] * 63
    n, per = ops.decode_plan(lens, 0, 8, SMS)
    assert n > 1
    assert per >= _chunks(1500, 0)            # a short request fits one slice
    assert n * per >= _chunks(30000, 0)
    blocks = sum(-(-_chunks(kl, 0) // per) for kl in lens) * 8
    assert blocks <= 5 * SMS                  # and the step does not drown in blocks


def test_every_request_is_covered_under_random_lengths_and_windows():
    rng = random.Random(5)
    for _ in range(300):
        lens = [rng.choice([1, 63, 64, 65, rng.randrange(1, 40000)]) for _ in range(rng.randrange(1, 70))]
        window = rng.choice([0, 0, 1, 100, 4096])
        f = rng.choice([1, 2, 8, 16])
        n, per = ops.decode_plan(lens, window, f, SMS)
        assert n in ops.DECODE_SLICE_COUNTS and per >= 1
        assert n * per >= max(_chunks(kl, window) for kl in lens)
        assert n == 1 or per >= 4
