"""The optional hand-over of additions and norms between parts, as far as it can be seen without a
GPU: parts that know nothing of it are left alone, and a norm takes back only what was made for it."""

import pytest
import torch

from mini_infer_b200.parts import (Arrangement, DeferredNorm, FeedForward, Mixer, Norm, PartSpec, StreamSink,
                                   build_part)


def _spec(kind, **params):
    return PartSpec(kind, dict(params), "")


def test_parts_say_no_unless_they_know_better():
    class ToyMixer(Mixer):
        pass

    class ToyFeedForward(FeedForward):
        pass

    class ToyNorm(Norm):
        pass

    class ToyBlock(Arrangement):
        pass

    m, f, n = ToyMixer(_spec("toy")), ToyFeedForward(_spec("toy")), ToyNorm(_spec("toy"))
    for rows in (1, 8, 16, 4096):
        assert not m.takes_deferred_norm(rows, "rms") and not m.adds_to_stream(rows, "rms")
        assert not f.takes_deferred_norm(rows, "rms") and not f.adds_to_stream(rows, "rms")
        assert n.stream_sink(torch.zeros(rows, 8), rows) is None and n.deferred_kind is None
    assert ToyBlock(m, f, n, n, None).entry() is None


def test_the_built_in_block_offers_its_entry_and_falls_back_without_a_gpu():
    norm = build_part("norm", _spec("rmsnorm", hidden_size=16, eps=1e-5))
    norm.bind({"weight": torch.ones(16)}, torch.float32, torch.device("cpu"))
    # on the CPU (or in float32) there is no fused form: the norm hands out no sink
    assert norm.stream_sink(torch.zeros(2, 16), 2) is None
    assert norm.stream_sink(None, 2) is None
    from mini_infer_b200.parts.builtin import PreNormBlock

    mixer = build_part("mixer", _spec("gqa_attention", hidden_size=32, num_heads=2, num_kv_heads=1, head_dim=16))
    ffn = build_part("feed_forward", _spec("swiglu", hidden_size=32, intermediate_size=48))
    block = PreNormBlock(mixer, ffn, norm, norm, None)
    assert block.entry() == (norm, mixer)


def test_a_norm_takes_back_only_what_was_made_for_it():
    a = build_part("norm", _spec("rmsnorm", hidden_size=16, eps=1e-5))
    b = build_part("norm", _spec("rmsnorm", hidden_size=16, eps=1e-5))
    stream = torch.zeros(2, 16)
    handed = DeferredNorm(a, "rms", torch.zeros(2, 16), object(), stream)
    x, residual = a.forward(handed, None)
    assert x is handed and residual is stream
    with pytest.raises(ValueError, match="another norm"):
        b.forward(handed, None)
    sink = StreamSink(a, "rms", stream, ("gain", 1e-5))
    assert a.deferred_kind == "rms" and sink.kind == "rms"
    assert sink.norm is a and sink.residual is stream and handed.shape == (2, 16) and handed.dtype == torch.float32
