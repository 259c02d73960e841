"""Configuration parsing, its refusals, and the architecture registry."""

import json

import pytest

from mini_infer_b200.config import (ConfigError, LlamaConfig, known_architectures, load_config,
                                    lookup_architecture, register_architecture, unregister_architecture)
from tiny_configs import TINY_A, TINY_B


def test_reads_every_size_from_config_json():
    a, b = LlamaConfig.from_json(TINY_A), LlamaConfig.from_json(TINY_B)
    assert (a.vocab_size, a.hidden_size, a.intermediate_size, a.num_hidden_layers) == (512, 64, 176, 2)
    assert (a.num_attention_heads, a.num_key_value_heads, a.head_dim, a.rms_norm_eps) == (4, 2, 16, 1e-5)
    assert a.rope_scaling.factor == 8.0 and a.rope_scaling.original_max_position_embeddings == 64
    assert not a.tie_word_embeddings and a.max_position_embeddings == 512
    assert (b.vocab_size, b.hidden_size, b.head_dim, b.rope_theta) == (1000, 192, 32, 500000.0)
    assert b.rope_scaling is None and b.tie_word_embeddings and b.rms_norm_eps == 1e-6
    for field in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
        assert getattr(a, field) != getattr(b, field)
    assert a.num_attention_heads // a.num_key_value_heads != b.num_attention_heads // b.num_key_value_heads


def test_defaults_and_alternative_keys():
    raw = dict(TINY_B)
    raw.pop("rope_scaling")
    raw.pop("rope_theta")
    assert LlamaConfig.from_json(raw).rope_theta == 10000.0
    raw["num_key_value_heads"] = None
    raw.pop("head_dim")
    cfg = LlamaConfig.from_json(raw)
    assert cfg.head_dim == 192 // 6 and cfg.num_key_value_heads == 6
    raw["rope_parameters"] = {"rope_theta": 123.0, "rope_type": "default"}
    assert LlamaConfig.from_json(raw).rope_theta == 123.0
    raw["rope_parameters"] = {"type": "llama3", "factor": 2.0, "low_freq_factor": 1.0,
                              "high_freq_factor": 4.0, "original_max_position_embeddings": 32}
    assert LlamaConfig.from_json(raw).rope_scaling.factor == 2.0


def test_round_trip_through_to_json():
    for raw in (TINY_A, TINY_B):
        cfg = LlamaConfig.from_json(raw)
        assert LlamaConfig.from_json(json.loads(json.dumps(cfg.to_json()))) == cfg


@pytest.mark.parametrize("kind", ["linear", "dynamic", "yarn"])
def test_other_rope_types_are_refused(kind):
    raw = dict(TINY_A, rope_scaling={"rope_type": kind, "factor": 2.0})
    with pytest.raises(NotImplementedError):
        LlamaConfig.from_json(raw)


def test_llama3_needs_all_fields_and_sane_values():
    base = dict(TINY_A["rope_scaling"])
    for missing in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings"):
        scaling = {k: v for k, v in base.items() if k != missing}
        with pytest.raises(ValueError, match=missing):
            LlamaConfig.from_json(dict(TINY_A, rope_scaling=scaling))
    for bad in ({"factor": 0.0}, {"high_freq_factor": 1.0}, {"original_max_position_embeddings": 0}):
        with pytest.raises(ValueError):
            LlamaConfig.from_json(dict(TINY_A, rope_scaling=dict(base, **bad)))


def test_biases_and_bad_sizes_are_refused():
    with pytest.raises(NotImplementedError):
        LlamaConfig.from_json(dict(TINY_A, attention_bias=True))
    with pytest.raises(NotImplementedError):
        LlamaConfig.from_json(dict(TINY_A, mlp_bias=True))
    with pytest.raises(ConfigError):
        LlamaConfig.from_json(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError):
        LlamaConfig.from_json({k: v for k, v in TINY_A.items() if k != "vocab_size"})
    with pytest.raises(ConfigError):
        LlamaConfig.from_json(dict(TINY_A, hidden_size="64"))


def test_registry_lookup_and_errors(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    arch, cfg = load_config(TINY_A)
    assert arch.name == "LlamaForCausalLM" and isinstance(cfg, LlamaConfig)
    with pytest.raises(ConfigError, match="registered"):
        lookup_architecture("NoSuchModel")
    with pytest.raises(ConfigError):
        load_config(dict(TINY_A, architectures=[]))
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(str(tmp_path))[1].hidden_size == 192
    with pytest.raises(FileNotFoundError):
        load_config(str(tmp_path / "nothing"))


def test_another_architecture_registers_without_touching_the_package():
    from mini_infer_b200.models.llama import assemble

    register_architecture("ToyLlamaTwin", LlamaConfig.from_json, assemble)
    try:
        with pytest.raises(ConfigError):
            register_architecture("ToyLlamaTwin", LlamaConfig.from_json, assemble)
        arch, cfg = load_config(dict(TINY_A, architectures=["ToyLlamaTwin"]))
        spec = arch.assemble(cfg)
        assert len(spec.layers) == 2 and spec.layers[0].mixer.kind == "gqa_attention"
    finally:
        unregister_architecture("ToyLlamaTwin")


def test_spec_schedule_rules():
    from mini_infer_b200.models.llama import assemble
    from mini_infer_b200.parts import ModelSpec, ScheduleEntry
    import dataclasses

    spec = assemble(LlamaConfig.from_json(TINY_A))
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1)]
    # a layer named twice, and a layer that reads another layer's cache
    twice = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
                                                ScheduleEntry(1, 0, writes_cache=False)))
    assert twice.num_cache_layers == 3
    with pytest.raises(ValueError):
        dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0)))
    with pytest.raises(ValueError):
        dataclasses.replace(spec, schedule=(ScheduleEntry(0, 1, writes_cache=False), ScheduleEntry(1, 1), ScheduleEntry(0, 0)))
    with pytest.raises(ValueError):
        dataclasses.replace(spec, schedule=(ScheduleEntry(5, 0),))
