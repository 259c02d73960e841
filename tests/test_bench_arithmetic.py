"""The byte and flop counts behind the benchmark's roofline fractions, checked against the
figures worked out by hand from the layer sizes (weights read once per decode step plus the
cache of the live requests; products and the causal half of attention for a prefill)."""

from __future__ import annotations

import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bench  # noqa: E402


def test_decode_bytes_of_the_8b_sizes():
    c = bench.LLAMA_8B
    # 32 layers x 218.1 M matrix parameters + the 525.3 M of the head, two bytes each,
    # and 128 KiB of keys and values per cached token
    assert bench.matmul_params(c, 32) == 32 * (4096 * 6144 + 4096 * 4096 + 3 * 4096 * 14336) + 128256 * 4096
    assert bench.decode_bytes(c, 32, 1, 2048) / 1e9 == pytest.approx(15.28, abs=0.01)
    assert bench.decode_bytes(c, 32, 8, 2048) / 1e9 == pytest.approx(17.16, abs=0.01)
    assert bench.decode_bytes(c, 32, 64, 2048) / 1e9 == pytest.approx(32.19, abs=0.01)
    per_token = bench.decode_bytes(c, 32, 1, 2049) - bench.decode_bytes(c, 32, 1, 2048)
    assert per_token == 128 * 1024


def test_prefill_flops_of_the_8b_sizes():
    c = bench.LLAMA_8B
    assert bench.prefill_flops(c, 32, 2048) / 1e13 == pytest.approx(2.97, abs=0.01)
    # attention alone: the causal half of 4 T^2 heads head_dim per layer
    only_attention = bench.prefill_flops(c, 32, 2048) - bench.prefill_flops(dict(c, num_attention_heads=0), 32, 2048)
    assert only_attention > 32 * 2.0 * 2048 * 2048 * 32 * 128


def test_the_70b_sizes():
    c = bench.LLAMA_70B
    assert c["hidden_size"] == 8192 and c["num_attention_heads"] == 64 and c["num_key_value_heads"] == 8
    assert bench.decode_bytes(c, 80, 8, 4096) / 1e9 == pytest.approx(149.7, abs=0.1)
    assert bench.prefill_flops(c, 80, 2048) / 1e14 == pytest.approx(2.86, abs=0.01)


def test_more_than_one_gpu_is_refused(capsys, monkeypatch):
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "2"])
    assert bench.main() == 2
    assert "one GPU" in capsys.readouterr().out
