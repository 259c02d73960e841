"""Safetensors I/O, binding by name with one clear error, dtype policy, random weights."""

import json
import os

import pytest
import torch

from mini_infer_b200.config import load_config
from mini_infer_b200.parts import DecoderModel
from mini_infer_b200.weights import (Checkpoint, SafetensorsError, WeightLoadError, check_names,
                                     random_state_dict, to_engine_dtype, write_random_model,
                                     write_safetensors)
from tiny_configs import TINY_A, TINY_B


def model_for(raw):
    arch, cfg = load_config(raw)
    return DecoderModel(arch.assemble(cfg))


def test_safetensors_round_trip_against_the_library(tmp_path):
    tensors = {
        "a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).view(2, 3),
        "d": torch.randn(2, 2).to(torch.float16), "e": torch.empty(0, 4), "f": torch.tensor(3.5),
    }
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors, metadata={"k": "v"})
    import safetensors.torch as st

    theirs = st.load_file(path)
    with Checkpoint(str(tmp_path)) as ck:
        assert sorted(ck.names()) == sorted(tensors)
        for n, t in tensors.items():
            mine = ck.read(n)
            assert mine.dtype == t.dtype and mine.shape == t.shape
            assert torch.equal(mine, t) and torch.equal(theirs[n], t)
    st.save_file({k: v for k, v in tensors.items()}, str(tmp_path / "lib.safetensors"))
    os.replace(str(tmp_path / "lib.safetensors"), path)
    with Checkpoint(str(tmp_path)) as ck:
        assert all(torch.equal(ck.read(n), t) for n, t in tensors.items())


def test_sharded_index_and_missing_files(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"x": torch.ones(2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"y": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    with Checkpoint(str(tmp_path)) as ck:
        assert sorted(ck.names()) == ["x", "y"] and ck.read("y").shape == (3,)
    with pytest.raises(FileNotFoundError):
        Checkpoint(str(tmp_path / "empty"))
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "model.safetensors").write_bytes(b"\x00\x01")
    with pytest.raises(SafetensorsError):
        Checkpoint(str(bad))


def test_expected_names_are_the_hugging_face_names():
    names = {e.name for e in model_for(TINY_A).expected_tensors()}
    assert "model.embed_tokens.weight" in names and "lm_head.weight" in names and "model.norm.weight" in names
    for part in ("input_layernorm", "post_attention_layernorm", "self_attn.q_proj", "self_attn.k_proj",
                 "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"):
        assert f"model.layers.1.{part}.weight" in names
    assert len(names) == 3 + 2 * 9
    tied = model_for(TINY_B)
    assert "lm_head.weight" not in {e.name for e in tied.expected_tensors()}
    assert tied.ignorable_tensors() == {"lm_head.weight"}


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    model = model_for(TINY_A)
    shapes = {e.name: e.decl.shape for e in model.expected_tensors()}
    check_names(model, shapes)
    broken = dict(shapes)
    del broken["model.layers.0.mlp.up_proj.weight"]
    del broken["lm_head.weight"]
    broken["extra.weight"] = (1,)
    broken["model.norm.weight"] = (65,)
    with pytest.raises(WeightLoadError) as info:
        check_names(model, broken)
    e = info.value
    assert e.missing == ["lm_head.weight", "model.layers.0.mlp.up_proj.weight"]
    assert e.unexpected == ["extra.weight"]
    assert e.mismatched == [("model.norm.weight", (64,), (65,))]
    text = str(e)
    for needle in ("missing", "unexpected", "wrong shape", "extra.weight", "expected (64,), found (65,)"):
        assert needle in text
    # a tied model tolerates a checkpoint that also ships the head
    tied = model_for(TINY_B)
    shapes = {e.name: e.decl.shape for e in tied.expected_tensors()}
    check_names(tied, dict(shapes, **{"lm_head.weight": (1000, 192)}))


def test_dtype_policy():
    bf, f32 = torch.bfloat16, torch.float32
    assert to_engine_dtype(torch.ones(2, dtype=bf), bf).dtype == bf
    assert to_engine_dtype(torch.ones(2, dtype=torch.float16), bf).dtype == bf
    assert to_engine_dtype(torch.ones(2, dtype=f32), bf).dtype == f32          # stored 32-bit stays
    assert to_engine_dtype(torch.ones(2, dtype=torch.int64), bf).dtype == torch.int32
    assert to_engine_dtype(torch.ones(2, dtype=bf), f32).dtype == f32
    x = torch.randn(100).to(bf)
    assert torch.equal(to_engine_dtype(x, f32), x.float())


def test_random_weights_are_seeded_and_shaped(tmp_path):
    s1 = random_state_dict(TINY_A, 5)
    s2 = random_state_dict(TINY_A, 5)
    s3 = random_state_dict(TINY_A, 6)
    assert all(torch.equal(s1[n], s2[n]) for n in s1)
    assert not torch.equal(s1["lm_head.weight"], s3["lm_head.weight"])
    assert s1["model.norm.weight"].float().mean().item() == pytest.approx(1.0, abs=0.05)
    assert s1["lm_head.weight"].float().std().item() == pytest.approx(0.02, rel=0.1)
    assert all(t.dtype == torch.bfloat16 for t in s1.values())
    out = write_random_model(TINY_B, str(tmp_path / "m"), 9)
    assert load_config(out)[1].hidden_size == 192
    with Checkpoint(out) as ck:
        model = model_for(TINY_B)
        check_names(model, {n: ck.shape(n) for n in ck.names()})
        assert ck.dtype("model.embed_tokens.weight") == torch.bfloat16


def test_random_generator_is_counter_based_and_exact():
    """The stream of a tensor depends on (seed, name, element index) only: the integer hash
    agrees with the same formula on Python integers (so nothing hangs on how a device wraps
    int64 products), a tensor drawn in pieces equals the tensor drawn at once, and the values
    are normal with the asked width."""
    from mini_infer_b200.weights import random_init as R

    key = R.tensor_seed(5, "model.layers.0.mlp.up_proj.weight")
    assert key == R.tensor_seed(5, "model.layers.0.mlp.up_proj.weight") != R.tensor_seed(6, "model.layers.0.mlp.up_proj.weight")
    index = torch.tensor([0, 1, 2, 12345, 2 ** 31, 2 ** 40 + 17], dtype=torch.int64)
    got = R.hash_bits(key, index).tolist()
    for i, g in zip(index.tolist(), got):
        assert g & ((1 << 64) - 1) == R.hash_bits_exact(key, i)
    whole = R.standard_normal(key, 0, 5000)
    pieces = torch.cat([R.standard_normal(key, 0, 1234), R.standard_normal(key, 1234, 5000 - 1234)])
    assert torch.equal(whole, pieces)
    z = R.standard_normal(key, 0, 200_000)
    assert abs(z.mean().item()) < 0.01 and abs(z.std().item() - 1.0) < 0.01
    assert abs((z ** 4).mean().item() - 3.0) < 0.1                      # a normal's fourth moment
    assert abs(((z.abs() > 1.959964).double().mean().item()) - 0.05) < 0.003
    assert abs((z[:-1] * z[1:]).mean().item()) < 0.01                   # neighbours do not correlate
    # the series used instead of library functions are accurate to a few ulps
    x = torch.rand(10_000, dtype=torch.float64) * 4e9 + 0.5
    assert (R._log_of(x) - torch.log(x)).abs().max().item() < 1e-13
    a = torch.linspace(0, 3.141592653589793 / 2, 10_001, dtype=torch.float64)
    assert (R._sin_quarter(a) - torch.sin(a)).abs().max().item() < 1e-14
    r = torch.rand(10_000, dtype=torch.float64) * 45 + 1e-10
    assert ((R._sqrt_of(r) - torch.sqrt(r)).abs() / torch.sqrt(r)).max().item() < 1e-15
    # a tensor larger than one chunk is drawn chunk by chunk and comes out the same
    t = R.random_tensor(1, "t", (3, 70_001), "matrix", std=0.02, gain_std=0.1)
    old, R._CHUNK = R._CHUNK, 4096
    try:
        assert torch.equal(R.random_tensor(1, "t", (3, 70_001), "matrix", std=0.02, gain_std=0.1), t)
    finally:
        R._CHUNK = old
    g = R.random_tensor(1, "g", (1000,), "gain", std=0.02, gain_std=0.1)
    assert abs(g.mean().item() - 1.0) < 0.02 and abs(g.std().item() - 0.1) < 0.02


@pytest.mark.gpu
def test_random_weights_are_the_same_on_cpu_and_gpu():
    """Bit for bit, in float32 and in bfloat16, for a matrix of odd size and a gain."""
    from mini_infer_b200.weights import random_init as R

    for shape, role in (((513, 1031), "matrix"), ((4097,), "gain"), ((1 << 22) + 5, "matrix")):
        shape = shape if isinstance(shape, tuple) else (shape,)
        for dtype in (torch.float32, torch.bfloat16):
            cpu = R.random_tensor(7, "w", shape, role, std=0.02, gain_std=0.1, dtype=dtype)
            gpu = R.random_tensor(7, "w", shape, role, std=0.02, gain_std=0.1, dtype=dtype, device="cuda:0")
            assert torch.equal(cpu, gpu.cpu()), (shape, role, dtype)
    key = R.tensor_seed(7, "w")
    assert torch.equal(R.standard_normal(key, 10, 100_000), R.standard_normal(key, 10, 100_000, "cuda:0").cpu())
