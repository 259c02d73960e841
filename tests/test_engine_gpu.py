"""Generation through the entry points, each part alone, and the generality of the parts
design: a toy mixer with state of its own, windows, a layer run twice, a shared cache."""

import dataclasses
import math
import os
import subprocess
import sys
import json
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_impl as P
import trace_util as T
from tiny_configs import PAGE_SIZE, TINY, load_state, prompt_ids

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ----------------------------------------------------------------------------- generation


@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_entry_point(which, model_dirs):
    from mini_infer_b200.engine import ContinuousScheduler, ModelRunner, Request
    from mini_infer_b200.sampling import SamplingParams

    state = load_state(model_dirs[which])
    lengths = {"A": [1, 17, 48], "B": [1, 7, 63, 130]}[which]
    n_new = {"A": 16, "B": 10}[which]
    prompts = [prompt_ids(which, n, salt=50 + i) for i, n in enumerate(lengths)]
    want = [P.greedy_generate(state, TINY[which], p, n_new) for p in prompts]
    runner = ModelRunner.from_pretrained(model_dirs[which], dtype="float32", block_size=PAGE_SIZE[which],
                                         num_blocks=96, max_requests=4)
    # a small token budget, so that prompt portions and decoded tokens share steps
    sched = ContinuousScheduler(runner, max_tokens_per_step=64 if which == "B" else 24, chunk_size=40)
    got = sched.generate([Request(p, SamplingParams(), n_new) for p in prompts])
    assert [r.tokens for r in got] == want
    assert all(r.finish_reason == "length" for r in got)
    assert runner.cache.num_free_pages() == 96


def test_generate_ids_and_command_line(model_dirs, tmp_path):
    from mini_infer_b200.engine.api import generate_ids

    state = load_state(model_dirs["A"])
    prompt = prompt_ids("A", 9, salt=77)
    want = P.greedy_generate(state, TINY["A"], prompt, 5)
    assert generate_ids(model_dirs["A"], [prompt], max_tokens=5, dtype="float32") == [want]
    out = subprocess.run(
        [sys.executable, "-m", "mini_infer_b200.generate", "--model", model_dirs["A"], "--dtype", "float32",
         "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--num-blocks", "16"],
        capture_output=True, text=True, cwd=T.ROOT, timeout=600)
    assert out.returncode == 0, out.stderr
    assert json.loads(out.stdout.strip().splitlines()[-1])["tokens"] == want


def test_sampling_is_seeded_and_independent_of_batching(model_dirs):
    from mini_infer_b200.engine import ContinuousScheduler, ModelRunner, Request
    from mini_infer_b200.sampling import SamplingParams

    which = "B"
    prompts = [prompt_ids(which, n, salt=90 + i) for i, n in enumerate([1, 7, 63, 130, 200])]
    params = [SamplingParams(temperature=0.8, seed=1000 + i) for i in range(5)]
    runner = ModelRunner.from_pretrained(model_dirs[which], dtype="float32", block_size=8, num_blocks=160,
                                         max_requests=5)

    def run(order, budget):
        sched = ContinuousScheduler(runner, max_tokens_per_step=budget, chunk_size=budget)
        res = sched.generate([Request(prompts[i], params[i], 24) for i in order])
        return {i: r.tokens for i, r in zip(order, res)}

    together = run([0, 1, 2, 3, 4], 64)
    again = run([0, 1, 2, 3, 4], 64)
    assert together == again
    alone = {}
    for i in range(5):
        alone.update(run([i], 512))
    assert together == alone              # fp32 logits do not depend on the batch, nor does the noise
    other_seed = ContinuousScheduler(runner).generate(
        [Request(prompts[3], SamplingParams(temperature=0.8, seed=5), 24)])[0].tokens
    assert other_seed != together[3]
    # the drawn tokens follow the plain implementation's logits
    state = load_state(model_dirs[which])
    seq = prompts[2] + together[2]
    logits = P.llama_logits(state, TINY[which], seq[:-1]).numpy()
    for n, tok in enumerate(together[2]):
        row = logits[len(prompts[2]) - 1 + n]
        ref_tok, score, keep = P.sample_reference(row, 0.8, 0, 1.0, params[2].seed, n)
        assert score[tok] >= score.max() - 1e-3


@pytest.mark.parametrize("cuda_graph", [False, True])
def test_decode_lookahead_gives_the_same_tokens(model_dirs, cuda_graph):
    """Launching the next decode step from the sampler's device output, before the host has
    read it, changes nothing but the time: same tokens with and without, with a stop token
    that ends one request early (its step ahead is thrown away and its pages come back)."""
    from mini_infer_b200.engine import ContinuousScheduler, ModelRunner, Request
    from mini_infer_b200.sampling import SamplingParams

    which = "A"
    prompts = [prompt_ids(which, n, salt=70 + i) for i, n in enumerate([9, 33, 50])]
    params = [SamplingParams(), SamplingParams(temperature=0.7, seed=11), SamplingParams(temperature=1.1, top_k=20, seed=12)]
    runner = ModelRunner.from_pretrained(model_dirs[which], dtype="bfloat16", block_size=16, num_blocks=40,
                                         max_requests=3, cuda_graph=cuda_graph)
    free = runner.cache.num_free_pages()

    def run(lookahead, eos=()):
        sched = ContinuousScheduler(runner, lookahead=lookahead, eos_token_ids=eos, chunk_size=64,
                                    max_tokens_per_step=128)
        res = sched.generate([Request(p, sp, 20) for p, sp in zip(prompts, params)])
        assert runner.cache.num_free_pages() == free and runner.cache.num_requests == 0
        return [r.tokens for r in res], [r.finish_reason for r in res], sched

    plain_tokens, _, _ = run(False)
    ahead_tokens, _, sched = run(True)
    assert ahead_tokens == plain_tokens
    assert sched.wasted_tokens == 0
    stop = plain_tokens[1][7]          # make the eighth token of the second request a stop token
    plain_tokens, plain_why, _ = run(False, eos=[stop])
    ahead_tokens, ahead_why, sched = run(True, eos=[stop])
    assert ahead_tokens == plain_tokens and ahead_why == plain_why
    assert "stop" in ahead_why and sched.wasted_tokens >= 1


@pytest.mark.parametrize("which", ["B", "C"])
def test_norms_ride_on_the_products_in_small_steps(which, model_dirs, monkeypatch):
    """In a bfloat16 step of a few tokens the blocks' additions and norms are done by the
    products around them: only the first norm and the final norm launch a kernel.  The logits
    agree with the route that launches every norm, and with the plain implementation."""
    from mini_infer_b200.csrc import ops
    from mini_infer_b200.engine import ModelRunner, StepEntry

    cfg = TINY[which]
    layers = cfg["num_hidden_layers"]
    prompt = prompt_ids(which, 37, salt=91)
    tail = prompt_ids(which, 6, salt=92)
    calls = []
    real = ops.add_rmsnorm

    def counting(*args, **kwargs):
        calls.append(1)
        return real(*args, **kwargs)

    monkeypatch.setattr(ops, "add_rmsnorm", counting)

    def run(fused):
        monkeypatch.setenv("MINI_INFER_FUSED_NORMS", "1" if fused else "0")
        runner = ModelRunner.from_pretrained(model_dirs[which], dtype="bfloat16", block_size=PAGE_SIZE[which],
                                             num_blocks=64, max_requests=2, cuda_graph=False)
        runner.add_request("r")
        runner.step([StepEntry("r", prompt, [])])
        rows, counts = [], []
        for tok in tail[:3]:
            del calls[:]
            rows.append(runner.step([StepEntry("r", [tok], [0])]).logits[0].float().cpu())
            counts.append(len(calls))
        del calls[:]
        rows.extend(runner.step([StepEntry("r", tail[3:], [0, 1, 2])]).logits.float().cpu())   # a portion of three
        counts.append(len(calls))
        return torch.stack(rows), counts

    fused, n_fused = run(True)
    unfused, n_unfused = run(False)
    assert n_unfused == [2 * layers + 1] * 4
    assert n_fused == [2] * 4
    # a norm of a kind the products do not know keeps its kernel, whatever the switch says
    from mini_infer_b200.parts.builtin import RMSNorm
    monkeypatch.setattr(RMSNorm, "deferred_kind", "a kind of its own")
    other, n_other = run(True)
    monkeypatch.undo()
    assert n_other == [2 * layers + 1] * 4 and torch.equal(other, unfused)
    want = P.llama_logits(load_state(model_dirs[which]), cfg, prompt + tail, dtype=torch.float64)[len(prompt):]
    bound = T.tolerance("bfloat16", float(want.abs().max()))
    for got in (fused, unfused):
        assert T.first_bad(got.double().numpy(), want.numpy(), bound) is None
    assert ops.gemm_tma_status() == 0


def test_decode_steps_of_every_batch_size_are_captured_ahead(model_dirs):
    """``capture_decode_steps`` leaves a graph per batch size and an empty cache behind, and what
    is generated afterwards (replaying those graphs from the first decode step on) is what the
    uncaptured engine generates."""
    from mini_infer_b200.engine import ContinuousScheduler, ModelRunner, Request
    from mini_infer_b200.sampling import SamplingParams

    prompts = [prompt_ids("C", n, salt=70 + i) for i, n in enumerate([9, 33, 5])]
    plain = ModelRunner.from_pretrained(model_dirs["C"], dtype="bfloat16", num_blocks=32, block_size=16, max_requests=4)
    want = [r.tokens for r in ContinuousScheduler(plain).generate([Request(p, SamplingParams(), 12) for p in prompts])]
    runner = ModelRunner.from_pretrained(model_dirs["C"], dtype="bfloat16", num_blocks=32, block_size=16, max_requests=4,
                                         cuda_graph=True)
    free = runner.cache.num_free_pages()
    assert runner.capture_decode_steps(4) == 4
    assert sorted(runner.stepper._graphs) == [(1,), (2,), (3,), (4,)]
    assert runner.cache.num_requests == 0 and runner.cache.num_free_pages() == free
    assert runner.capture_decode_steps(4) == 0          # nothing left to capture
    replays = sum(slot.replays for slot in runner.stepper._graphs.values())
    got = [r.tokens for r in ContinuousScheduler(runner).generate([Request(p, SamplingParams(), 12) for p in prompts])]
    assert got == want
    assert sum(slot.replays for slot in runner.stepper._graphs.values()) > replays
    runner.cache.check()


def test_engine_thread_streams_the_same_tokens(model_dirs):
    """The engine loop on a thread of its own (``start`` / ``stop``): requests submitted from
    this thread while it runs, tokens streamed through callbacks, the runner's health word read
    with every step; same tokens as the plain implementation."""
    from mini_infer_b200.engine import ContinuousScheduler, ModelRunner, Request
    from mini_infer_b200.sampling import SamplingParams

    which = "C"
    state = load_state(model_dirs[which])
    prompts = [prompt_ids(which, n, salt=20 + i) for i, n in enumerate([30, 5, 70])]
    want = [P.greedy_generate(state, TINY[which], p, 12) for p in prompts]
    for dtype, graph in (("float32", False), ("bfloat16", True)):
        runner = ModelRunner.from_pretrained(model_dirs[which], dtype=dtype, block_size=16, num_blocks=32,
                                             max_requests=4, cuda_graph=graph)
        sched = ContinuousScheduler(runner, chunk_size=32, max_tokens_per_step=48)
        sched.start()
        try:
            streamed = [[] for _ in prompts]
            handles = [sched.submit(Request(p, SamplingParams(), 12), on_token=streamed[i].append)
                       for i, p in enumerate(prompts)]
            results = [h.wait(timeout=300) for h in handles]
        finally:
            sched.stop()
        assert [r.tokens for r in results] == streamed
        assert all(r.finish_reason == "length" for r in results)
        if dtype == "float32":
            assert streamed == want
        assert int(runner.health_word().item()) == 0
        assert runner.cache.num_requests == 0 and runner.cache.num_free_pages() == 32


def test_preemption_by_recompute_gives_the_same_tokens(model_dirs):
    from mini_infer_b200.engine import ContinuousScheduler, ModelRunner, Request
    from mini_infer_b200.sampling import SamplingParams

    which = "A"
    state = load_state(model_dirs[which])
    prompts = [prompt_ids(which, 40, salt=3), prompt_ids(which, 35, salt=4)]
    want = [P.greedy_generate(state, TINY[which], p, 30) for p in prompts]
    runner = ModelRunner.from_pretrained(model_dirs[which], dtype="float32", block_size=16, num_blocks=8,
                                         max_requests=2)
    sched = ContinuousScheduler(runner, decode_headroom_blocks=0, chunk_size=64, max_tokens_per_step=128)
    got = sched.generate([Request(p, SamplingParams(), 30) for p in prompts])
    assert sched.preemptions >= 1
    assert [r.tokens for r in got] == want
    assert runner.cache.num_free_pages() == 8


# ----------------------------------------------------------------------------- parts alone


def stub_runner(cache, dtype, tile_sizes=(16,), vocab=100):
    from mini_infer_b200.engine.step import StepRunner
    from mini_infer_b200.parts import PlanNeeds

    model = SimpleNamespace(device=torch.device(DEV), dtype=dtype,
                            spec=SimpleNamespace(vocab_size=vocab, max_positions=None),
                            plan_needs=lambda: PlanNeeds(frozenset(tile_sizes)), schedule=())
    return StepRunner(model, cache)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_alone_in_portions(dtype):
    """The mixer part by itself (own sizes: 5 heads over 1 key/value head of 48), fed a
    sequence in portions through a real cache, against plain whole-sequence attention."""
    from mini_infer_b200.cache import CacheManager
    from mini_infer_b200.engine.step import StepEntry
    from mini_infer_b200.parts import LayerCache, PartSpec, build_part

    H, nq, nkv, d, Tn = 72, 5, 1, 48, 45
    mixer = build_part("mixer", PartSpec("gqa_attention", {"hidden_size": H, "num_heads": nq,
                                                           "num_kv_heads": nkv, "head_dim": d}))
    rope = build_part("position", PartSpec("rotary", {"head_dim": d, "theta": 1234.0}))
    g = torch.Generator().manual_seed(0)
    w = {n: (torch.randn(*decl.shape, generator=g) * (0.2 if "q_" in n or "k_" in n else 0.1)).to(torch.bfloat16)
         for n, decl in mixer.param_decls().items()}
    mixer.bind({n: t.to(DEV) for n, t in w.items()}, dtype, torch.device(DEV))
    rope.bind({}, dtype, torch.device(DEV))
    need = SimpleNamespace(index=0, kv=mixer.cache_need(), state=None)
    cache = CacheManager([need], page_size=4, num_pages=16, max_requests=1, dtype=dtype, device=DEV)
    runner = stub_runner(cache, dtype, tile_sizes=mixer.plan_needs().q_tile_tokens)
    x = (torch.randn(Tn, H, generator=g)).to(torch.bfloat16)
    cache.add_request("r")
    outs, pos = [], 0
    for n in (7, 1, 2, 19, 16):
        ctx, _, _, _ = runner.plan([StepEntry("r", [0] * n, [])])
        runner.apply_table_updates(ctx)
        gi, k, v = cache.layer_kv(0)
        out = mixer.forward(x[pos:pos + n].to(DEV).to(dtype), ctx, LayerCache(group=gi, k=k, v=v), rope)
        outs.append(out.float().cpu())
        pos += n
    got = torch.cat(outs).double()
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d}
    cos, sin = P.rope_cos_sin(list(range(Tn)), P.rope_inv_freq(d, 1234.0, None), torch.float64)
    want = P.attention_block(x.double(), {k: t.double() for k, t in w.items()}, "", cfg, cos, sin)
    bound = (1e-4 if dtype == torch.float32 else 3e-2) * want.abs().max().item()
    assert (got - want).abs().max().item() <= bound


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_norm_embedding_head_parts_alone(dtype):
    from mini_infer_b200.parts import PartSpec, build_part

    dev = torch.device(DEV)
    H, I, V, M = 136, 200, 333, 9
    g = torch.Generator().manual_seed(1)
    rel = 1e-4 if dtype == torch.float32 else 3e-2
    ffn = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}))
    w = {n: (torch.randn(*d.shape, generator=g) * 0.1).to(torch.bfloat16) for n, d in ffn.param_decls().items()}
    ffn.bind({n: t.to(DEV) for n, t in w.items()}, dtype, dev)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16)
    got = ffn.forward(x.to(DEV).to(dtype), None).float().cpu().double()
    want = P.swiglu(x.double(), w["gate_proj.weight"].double(), w["up_proj.weight"].double(),
                    w["down_proj.weight"].double())
    assert (got - want).abs().max().item() <= rel * want.abs().max().item()

    norm = build_part("norm", PartSpec("rmsnorm", {"hidden_size": H, "eps": 3e-4}))
    gain = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    norm.bind({"weight": gain.to(DEV)}, dtype, dev)
    res = torch.randn(M, H, generator=g)
    out, new_res = norm.forward(x.to(DEV).to(dtype), res.to(DEV))
    want = P.rms_norm(x.double() + res.double(), gain.double(), 3e-4)
    assert (out.float().cpu().double() - want).abs().max().item() <= rel * want.abs().max().item()
    assert torch.allclose(new_res.cpu().double(), x.double() + res.double(), atol=1e-6)
    first, res0 = norm.forward(x.to(DEV).to(dtype), None)
    assert torch.equal(res0.cpu(), x.float())

    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}))
    table = torch.randn(V, H, generator=g).to(torch.bfloat16)
    emb.bind({"weight": table.to(DEV)}, dtype, dev)
    ids = torch.tensor([0, V - 1, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(SimpleNamespace(token_ids=ids)).float().cpu(), table[ids.long().cpu()].float())
    head = build_part("head", PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "tied": True}))
    head.bind({}, dtype, dev, tied_weight=emb.weight)
    logits = head.forward(x.to(DEV).to(dtype))
    assert logits.dtype == torch.float32
    want = x.double() @ table.double().T
    assert (logits.cpu().double() - want).abs().max().item() <= rel * want.abs().max().item()


# ----------------------------------------------------------------------------- generality


def _register_toys():
    """Test-only parts and architectures; nothing in the package knows them."""
    from mini_infer_b200.config import register_architecture
    from mini_infer_b200.models.llama import assemble as llama_assemble
    from mini_infer_b200.config import LlamaConfig
    from mini_infer_b200.parts import (FeedForward, Mixer, ParamDecl, PartSpec, Position, ScheduleEntry, StateNeed,
                                       register_feed_forward, register_mixer, register_position)

    class RunningMeanMixer(Mixer):
        """out_t = W * mean(x_0 .. x_t): its state is the running sum and the count."""

        def param_decls(self):
            H = self.param("hidden_size")
            return {"mix.weight": ParamDecl((H, H))}

        def state_need(self):
            return StateNeed((self.param("hidden_size") + 1,), torch.float32)

        def bind(self, tensors, dtype, device):
            self.w = tensors["mix.weight"].float()

        def forward(self, x, ctx, cache, position):
            H = self.param("hidden_size")
            out = torch.empty_like(x)
            for start, n, slot in zip(ctx.host_q_start, ctx.host_q_len, ctx.host_state_slot):
                st = cache.state[slot]
                sums = st[:H] + torch.cumsum(x[start:start + n].float(), dim=0)
                counts = st[H] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[start:start + n] = ((sums / counts[:, None]) @ self.w.T).to(x.dtype)
                st[:H] = sums[-1]
                st[H] = counts[-1]
            return out

    RunningMeanMixer.graph_safe = False      # it reads the host lists of the step: never captured
    register_mixer("toy_running_mean", RunningMeanMixer, replace=True)

    class RunningMeanOnDevice(RunningMeanMixer):
        """The same mixer with a decode path that touches device tensors only (rows gathered and
        scattered by the step's slot indices), so a captured step may replay it."""

        graph_safe = True

        def forward(self, x, ctx, cache, position):
            if not ctx.decode_only:
                return super().forward(x, ctx, cache, position)
            H = self.param("hidden_size")
            slots = ctx.state_slot.long()
            st = cache.state.index_select(0, slots)
            sums = st[:, :H] + x.float()
            counts = st[:, H] + 1.0
            cache.state.index_copy_(0, slots, torch.cat([sums, counts[:, None]], dim=1))
            return ((sums / counts[:, None]) @ self.w.T).to(x.dtype)

    register_mixer("toy_running_mean_device", RunningMeanOnDevice, replace=True)

    class SoftRoutedExperts(FeedForward):
        """sum_e softmax(x R^T)_e * down_e(silu(up_e x)): a router (fp32 logits and softmax) and
        several experts of its own sizes; a feed-forward with routing, with plain torch ops."""

        def param_decls(self):
            H, I, E = self.param("hidden_size"), self.param("expert_size"), self.param("experts")
            decls = {"router.weight": ParamDecl((E, H))}
            for e in range(E):
                decls[f"experts.{e}.up.weight"] = ParamDecl((I, H))
                decls[f"experts.{e}.down.weight"] = ParamDecl((H, I))
            return decls

        def bind(self, tensors, dtype, device):
            self.t = {k: v.to(dtype) for k, v in tensors.items()}

        def forward(self, x, ctx):
            gates = torch.softmax(x.float() @ self.t["router.weight"].float().T, dim=-1)
            out = torch.zeros_like(x, dtype=torch.float32)
            for e in range(self.param("experts")):
                hidden = torch.nn.functional.silu((x @ self.t[f"experts.{e}.up.weight"].T).float()).to(x.dtype)
                out += gates[:, e:e + 1] * (hidden @ self.t[f"experts.{e}.down.weight"].T).float()
            return out.to(x.dtype)

    register_feed_forward("toy_soft_experts", SoftRoutedExperts, replace=True)

    class LearnedOffsets(Position):
        """q and k get a learned vector added that depends on the position modulo a period:
        another position encoding than rotation; keys are stored by the default store path."""

        def param_decls(self):
            return {"table": ParamDecl((self.param("period"), self.param("head_dim")))}

        def bind(self, tensors, dtype, device):
            self.table = tensors["table"].to(dtype)

        def encode(self, qkv, nq, nkv, head_dim, ctx):
            add = self.table[(ctx.positions.long() % self.param("period"))]          # [tokens, d]
            heads = qkv[:, : (nq + nkv) * head_dim].view(qkv.shape[0], nq + nkv, head_dim)
            heads += add[:, None, :]

    register_position("toy_learned_offsets", LearnedOffsets, replace=True)

    def toy_state_assemble(cfg, kind="toy_running_mean"):
        spec = llama_assemble(cfg)
        layers = list(spec.layers)
        layers[0] = dataclasses.replace(
            layers[0], position=None,
            mixer=PartSpec(kind, {"hidden_size": cfg.hidden_size}, prefix="model.layers.0.toy."))
        return dataclasses.replace(spec, layers=tuple(layers))

    def routed_assemble(cfg):
        spec = llama_assemble(cfg)
        layers = list(spec.layers)
        layers[1] = dataclasses.replace(
            layers[1],
            feed_forward=PartSpec("toy_soft_experts", {"hidden_size": cfg.hidden_size, "expert_size": 40, "experts": 3},
                                  prefix="model.layers.1.moe."),
            position=PartSpec("toy_learned_offsets", {"head_dim": cfg.head_dim, "period": 7},
                              prefix="model.layers.1.pos."))
        return dataclasses.replace(spec, layers=tuple(layers))

    def windowed_assemble(cfg):
        spec = llama_assemble(cfg)
        layers = list(spec.layers)
        for i in range(0, len(layers), 2):
            layers[i] = dataclasses.replace(
                layers[i], mixer=dataclasses.replace(layers[i].mixer, params=dict(layers[i].mixer.params, window=11)))
        return dataclasses.replace(spec, layers=tuple(layers))

    def looped_assemble(cfg):
        spec = llama_assemble(cfg)
        return dataclasses.replace(spec, schedule=(
            ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(1, 0, writes_cache=False)))

    register_architecture("ToyStateLM", LlamaConfig.from_json, toy_state_assemble, replace=True)
    register_architecture("ToyStateOnDeviceLM", LlamaConfig.from_json,
                          lambda cfg: toy_state_assemble(cfg, "toy_running_mean_device"), replace=True)
    register_architecture("ToyWindowLM", LlamaConfig.from_json, windowed_assemble, replace=True)
    register_architecture("ToyLoopLM", LlamaConfig.from_json, looped_assemble, replace=True)
    register_architecture("ToyRoutedLM", LlamaConfig.from_json, routed_assemble, replace=True)


def plain_variant(state, raw, ids, *, windows=None, schedule=None, toy_layers=(), routed_layers=()):
    """The plain decoder with per-layer windows, a run order and toy layers (float64)."""
    cfg = P.normalise_config(raw)
    w = {k: v.double() for k, v in state.items()}
    L = cfg["num_hidden_layers"]
    schedule = schedule or [(i, i, True) for i in range(L)]
    windows = windows or [None] * L
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    Tn = len(ids)
    cos, sin = P.rope_cos_sin(list(range(Tn)), P.rope_inv_freq(d, cfg["_theta"], cfg["_scaling"]), torch.float64)
    h = P.embed(w["model.embed_tokens.weight"], ids)
    kv_of = {}
    for layer, cache, writes in schedule:
        p = f"model.layers.{layer}."
        a = P.rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        if layer in toy_layers:
            mean = torch.cumsum(a, dim=0) / torch.arange(1, Tn + 1, dtype=torch.float64)[:, None]
            h = h + mean @ w[p + "toy.mix.weight"].T
        else:
            if layer in routed_layers:       # learned offsets by position modulo the period, no rotation
                table = w[p + "pos.table"]
                add = table[torch.arange(Tn) % table.shape[0]][:, None, :]
                encode = lambda t: t + add
            else:
                encode = lambda t: P.apply_rope(t, cos, sin)
            q = encode((a @ w[p + "self_attn.q_proj.weight"].T).view(Tn, nq, d))
            if writes:
                k = encode((a @ w[p + "self_attn.k_proj.weight"].T).view(Tn, nkv, d))
                v = (a @ w[p + "self_attn.v_proj.weight"].T).view(Tn, nkv, d)
                kv_of[cache] = (k, v)
            k, v = kv_of[cache]
            o = P.causal_attention(q, k, v, 1 / math.sqrt(d), windows[layer])
            h = h + o.reshape(Tn, nq * d) @ w[p + "self_attn.o_proj.weight"].T
        b = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        if layer in routed_layers:
            gates = torch.softmax(b @ w[p + "moe.router.weight"].T, dim=-1)
            for e in range(gates.shape[1]):
                hidden = P.silu(b @ w[p + f"moe.experts.{e}.up.weight"].T)
                h = h + gates[:, e:e + 1] * (hidden @ w[p + f"moe.experts.{e}.down.weight"].T)
        else:
            h = h + P.swiglu(b, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                             w[p + "mlp.down_proj.weight"])
    z = P.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return (z @ head.T).numpy()


def cut_prefill_then_decode(requests, n_decode):
    """Every request's prompt in a step of its own (no logits), then ``n_decode`` steps in which
    all of them bring one token: the steps a captured graph replays."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": rid, "tokens": toks[:-n_decode], "want": [len(toks) - n_decode - 1]}]})
    for i in range(n_decode):
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": rid, "tokens": [toks[len(toks) - n_decode + i]], "want": [0]}
                                  for rid, toks in requests.items()]})
    steps[-1]["end"] = list(requests)
    return steps


def run_variant(arch, raw_base, tmp_path, dtype, page, plain_kwargs, num_blocks=None, cuda_graph=False, which="A"):
    from mini_infer_b200.engine import ModelRunner
    from mini_infer_b200.weights import write_random_model
    from tiny_configs import PEAKED

    _register_toys()
    raw = dict(raw_base, architectures=[arch])
    # wide enough that a wrong offset, gate or expert would show in the logits
    wide = dict(PEAKED[which], **{"pos.table": 0.7, "router.weight": 0.5, "experts.": 0.08})
    folder = write_random_model(raw, str(tmp_path / arch), 5, std_overrides=wide)
    state = load_state(folder)
    requests = {f"q{i}": prompt_ids(which, n, salt=200 + i) for i, n in enumerate([50, 13 if cuda_graph else 3, 77, 31])}
    want = {r: plain_variant(state, raw, toks, **plain_kwargs) for r, toks in requests.items()}
    n_decode = 12
    steps = cut_prefill_then_decode(requests, n_decode) if cuda_graph else T.cut_mixed(requests, n_decode=9)
    runner = ModelRunner.from_pretrained(folder, dtype=dtype, block_size=page,
                                         num_blocks=num_blocks or T.max_tokens_needed(steps) // page, max_requests=4,
                                         cuda_graph=cuda_graph)
    for st in runner.cache.storage:
        st.fill_(float("nan"))
    got = T.collect(steps, T.replay_in_process(runner, steps), raw["vocab_size"])
    runner.cache.check()
    scale = max(float(np.abs(want[r]).max()) for r in want)
    for r in requests:
        # with graphs the trace asks for the last prompt position and the decoded ones only
        ref = want[r][-(n_decode + 1):] if cuda_graph else want[r]
        bad = T.first_bad(got[r], ref, T.tolerance(dtype, scale))
        assert bad is None, (f"{arch}/{dtype}: request {r} first differs at position {bad}: |diff| = "
                             f"{np.abs(got[r][bad] - ref[bad]).max():.3e}, largest over the request "
                             f"{np.abs(got[r] - ref).max():.3e}, logit scale {scale:.3f}")
    return runner


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_of_its_own(dtype, tmp_path):
    """A mixer defined here, with a per-request state slot, is registered, built, given
    weights by name and stepped in mixed batches, next to an attention layer."""
    runner = run_variant("ToyStateLM", TINY["A"], tmp_path, dtype, 16, {"toy_layers": (0,)})
    assert 0 in runner.cache.state_arenas and 1 not in runner.cache.state_arenas
    assert [g.layers for g in runner.cache.groups] == [(1,)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stateful_mixers_and_captured_steps(dtype, tmp_path):
    """``cuda_graph=True`` with mixers that keep a state of their own.  One whose decode path
    runs on device tensors only is captured and replayed, and its state advances exactly once
    per step, the first step of a kind included (that step runs kernel by kernel and is then
    captured without being run again).  One that reads the step's host lists says so
    (``graph_safe = False``): its model is never captured and still gives the right logits."""
    runner = run_variant("ToyStateOnDeviceLM", TINY["A"], tmp_path, dtype, 16, {"toy_layers": (0,)}, cuda_graph=True)
    assert sum(slot.replays for slot in runner.stepper._graphs.values()) >= 10
    runner = run_variant("ToyStateLM", TINY["A"], tmp_path, dtype, 16, {"toy_layers": (0,)}, cuda_graph=True)
    assert not runner.stepper.cuda_graph and not runner.stepper._graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_layers_in_captured_steps(dtype, tmp_path):
    """Decode steps of a model with windowed and full layers (two cache groups, the windowed
    one handing pages back while it decodes) replayed as captured graphs."""
    runner = run_variant("ToyWindowLM", TINY["A"], tmp_path, dtype, 4, {"windows": [11, None]},
                         num_blocks=[48, 80], cuda_graph=True)
    assert sum(slot.replays for slot in runner.stepper._graphs.values()) >= 10
    assert [(g.layers, g.window) for g in runner.cache.groups] == [((0,), 11), ((1,), None)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_another_position_encoding(dtype, tmp_path):
    """A feed-forward with a router and experts and a position encoding that is no rotation,
    both defined here, take the place of a layer's SwiGLU and rotary parts: registered, built,
    given their tensors by name, and stepped in mixed batches beside an ordinary layer."""
    runner = run_variant("ToyRoutedLM", TINY["A"], tmp_path, dtype, 16, {"routed_layers": (1,)})
    names = {t.name for t in runner.model.expected_tensors()}
    assert "model.layers.1.moe.router.weight" in names and "model.layers.1.pos.table" in names
    assert "model.layers.1.mlp.gate_proj.weight" not in names


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_and_without_a_window_have_pages_of_their_own(dtype, tmp_path):
    runner = run_variant("ToyWindowLM", TINY["A"], tmp_path, dtype, 4, {"windows": [11, None]},
                         num_blocks=[48, 80])
    assert [(g.layers, g.window) for g in runner.cache.groups] == [((0,), 11), ((1,), None)]


def test_decode_kernel_that_rotates_by_itself_in_windowed_and_shared_cache_layers(tmp_path):
    """At a head size the decode kernel takes (64), captured decode-only bfloat16 steps leave the
    rotation of q and the storing of the newest key and value to the attention kernel: with a
    windowed layer (its pages handed back while it decodes), and with a layer that only reads
    another layer's cache (q is rotated, nothing is stored)."""
    from mini_infer_b200.csrc import ops

    assert ops.decode_rope_fusable(torch.bfloat16, TINY["C"]["head_dim"], True, 4)
    runner = run_variant("ToyWindowLM", TINY["C"], tmp_path / "w", "bfloat16", 16, {"windows": [11, None]},
                         num_blocks=[48, 80], cuda_graph=True, which="C")
    assert sum(slot.replays for slot in runner.stepper._graphs.values()) >= 10
    runner = run_variant("ToyLoopLM", TINY["C"], tmp_path / "l", "bfloat16", 16,
                         {"schedule": [(0, 0, True), (1, 1, True), (0, 2, True), (1, 0, False)]}, cuda_graph=True, which="C")
    assert sum(slot.replays for slot in runner.stepper._graphs.values()) >= 10


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_run_twice_and_a_layer_reading_anothers_cache(dtype, tmp_path):
    run_variant("ToyLoopLM", TINY["A"], tmp_path, dtype, 16,
                {"schedule": [(0, 0, True), (1, 1, True), (0, 2, True), (1, 0, False)]})
