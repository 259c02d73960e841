"""Benchmark: decode and prefill throughput at Llama 3.1 8B layer sizes, random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests, each holding 2,048 tokens of context
(growing by one per step).  The one JSON line printed at the end carries:

``value``      decoded tokens per second at batch 8, timed on the device with CUDA events
               around exactly K steps (after W warm-up steps);
``e2e``        the same through the Python entry point (``ContinuousScheduler.step``): host
               token ids in (pinned staging, one host-to-device copy per step) and sampled
               ids read back to the host every step;
``prefill``    one 2,048-token prompt in one step: tokens/s, ms, and flops / time / peak;
``roofline``   bytes the decode step must read (every weight once, plus the cache of the
               live requests) / time, against the measured copy bandwidth;
``points``     decode tokens/s at batch 1 and 64;
``clocks``     SM clocks and throttle reasons sampled during the timed regions.

``--scenario serving`` is the workload the reference published numbers for (1,024-token
prompts, 128 generated tokens, five single requests and one batch of 16, through the
scheduler's engine thread; ``scripts/bench/modal_model_metrics.py:59-63,126-204``), for either
arm, as a line of its own.

Weights are far larger than L2, so nothing is flushed between timed iterations
(``config.l2``).  The engine is single-GPU: ``--gpus N`` with N > 1 prints one line and
exits with status 2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Layer sizes of Llama 3.1 8B (the benchmark's model; the engine itself reads sizes from
# config.json only).
LLAMA_8B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 128256,
    "hidden_size": 4096,
    "intermediate_size": 14336,
    "num_hidden_layers": 32,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072,
    "tie_word_embeddings": False,
}
# The same architecture at Llama 3.1 70B's layer sizes (a further measurement point,
# ``--sizes 70b``: 141 GB of weights, drawn on the device part by part; ``--context 4096`` is
# the context the benchmark's description names for it).
LLAMA_70B = dict(LLAMA_8B, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                 num_attention_heads=64)
SIZES = {"8b": ("Llama 3.1 8B", LLAMA_8B, 32), "70b": ("Llama 3.1 70B", LLAMA_70B, 80)}
POINTS = {"8b": (1, 64), "70b": (1,)}      # further batch sizes measured beside the headline's
CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE = 16
BASELINE_DECODE_TOK_S = 276.0   # the reference's published single-request decode speed on a B200


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p.get("bf16_tflops_sustained") or p["bf16_tflops"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi while a timed region runs (reads settings only)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self._proc = None
        self._thread = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return

        def pump() -> None:
            for line in self._proc.stdout:
                self.samples.append([c.strip() for c in line.split(",")])

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def matmul_params(cfg: dict, layers: int) -> int:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I
    return layers * per_layer + V * H


def decode_bytes(cfg: dict, layers: int, batch: int, context: int) -> float:
    nkv, d, H = cfg["num_key_value_heads"], cfg["head_dim"], cfg["hidden_size"]
    weights = 2.0 * (matmul_params(cfg, layers) + (2 * layers + 1) * H)
    cache = 2.0 * batch * context * 2 * nkv * d * layers
    return weights + cache + 2.0 * batch * H      # + the embedding rows read


def prefill_flops(cfg: dict, layers: int, tokens: int) -> float:
    nq, d, V, H = cfg["num_attention_heads"], cfg["head_dim"], cfg["vocab_size"], cfg["hidden_size"]
    gemm = 2.0 * tokens * (matmul_params(cfg, layers) - V * H) + 2.0 * V * H     # the head runs on one row
    attention = layers * 2.0 * tokens * tokens * nq * d                            # causal half of 4 T^2 nq d
    return gemm + attention


def build_runner(cfg: dict, layers: int, num_blocks: int, max_requests: int):
    import torch

    from mini_infer_b200.engine import ModelRunner

    raw = dict(cfg, num_hidden_layers=layers)
    runner = ModelRunner.from_random(raw, seed=0, gain_std=0.0, device="cuda:0", dtype="bfloat16",
                                     num_blocks=num_blocks, block_size=PAGE, max_requests=max_requests,
                                     cuda_graph=True)
    torch.cuda.empty_cache()
    return runner


def fill_cache(runner, batch: int, context: int) -> list[str]:
    """Admit ``batch`` requests that already hold ``context`` tokens of (random) keys and
    values: a decode step's cost does not depend on what the cache holds."""
    import torch

    for st in runner.cache.storage:
        st.normal_(0.0, 1.0)
    rids = []
    for i in range(batch):
        rid = f"bench{i}"
        runner.add_request(rid)
        runner.cache.plan_append([(rid, context)])
        rids.append(rid)
    torch.cuda.synchronize()
    return rids


def time_decode(runner, batch: int, context: int, steps: int, warmup: int) -> tuple[float, int]:
    """(milliseconds per decode step, kernels launched in the timed region), device-timed."""
    import torch

    from mini_infer_b200.csrc import ops
    from mini_infer_b200.engine import StepEntry
    from mini_infer_b200.sampling import DeviceSampler, SamplingParams

    rids = fill_cache(runner, batch, context)
    sampler = DeviceSampler(runner.device)
    params = [SamplingParams()] * batch
    gen = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, runner.vocab_size, (steps + warmup, batch), generator=gen).tolist()

    def one(i: int) -> None:
        res = runner.step([StepEntry(r, [tokens[i][j]], [0]) for j, r in enumerate(rids)])
        sampler.sample(res.logits, params, [0] * batch, [i] * batch)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches0 = ops.launch_count
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = ops.launch_count - launches0
    for r in rids:
        runner.free_request(r)
    return ms, launches


def time_prefill(runner, tokens: int, repeats: int, warmup: int) -> float:
    import torch

    from mini_infer_b200.engine import StepEntry

    gen = torch.Generator().manual_seed(2)
    ids = torch.randint(0, runner.vocab_size, (tokens,), generator=gen).tolist()
    times = []
    for i in range(warmup + repeats):
        runner.add_request("prefill")
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry("prefill", ids, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.free_request("prefill")
        if i >= warmup:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def time_e2e(runner, batch: int, context: int, steps: int, warmup: int) -> dict:
    """Decode through the scheduler: real prompts are prefilled (untimed), then K engine steps
    are timed by the wall clock with a device synchronise on both sides; every step copies its
    token ids from pinned host memory and reads the sampled ids back."""
    import torch

    from mini_infer_b200.engine import ContinuousScheduler, Request
    from mini_infer_b200.sampling import SamplingParams

    gen = torch.Generator().manual_seed(3)
    sched = ContinuousScheduler(runner, max_concurrent=batch, chunk_size=context,
                                max_tokens_per_step=max(context, batch), decode_headroom_blocks=0)
    for _ in range(batch):
        prompt = torch.randint(0, runner.vocab_size, (context,), generator=gen).tolist()
        sched.submit(Request(prompt, SamplingParams(), max_tokens=steps + warmup + 2 * batch + 8))
    while sched.has_prefill_work():
        sched.step()
    for _ in range(warmup):
        sched.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        sched.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    sched.stop()
    return {"value": batch * steps / dt, "unit": "tokens/s", "ms_per_step": 1000.0 * dt / steps,
            "h2d_bytes_per_step": runner.stepper.last_h2d_bytes, "d2h_bytes_per_step": 4 * batch}


def run_long_mixed(args) -> int:
    """The long mixed workload: ``--requests`` requests started together, prompt lengths drawn
    log-uniformly from [16, ``--max-prompt``], ``--generate`` greedy tokens each, a step budget
    of 2048 tokens, admission by free pages.  Prints one JSON line of its own (total tokens a
    second, step times, the pool's high-water mark, preemptions); it is no part of the
    contract line.  Timed by the wall clock with a device synchronise on both sides."""
    _, cfg, _ = SIZES[args.sizes]
    layers = args.layers
    token_bytes = 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    num_blocks = int(args.pool_gb * 1e9 / (token_bytes * PAGE))
    runner = build_runner(cfg, layers, num_blocks=num_blocks, max_requests=args.requests)
    print(json.dumps(long_mixed(runner, args, num_blocks)))
    return 0


def long_mixed(runner, args, num_blocks: int) -> dict:
    import math

    import torch

    from mini_infer_b200.engine import ContinuousScheduler, Request
    from mini_infer_b200.sampling import SamplingParams

    model_name, cfg, _ = SIZES[args.sizes]
    layers = args.layers
    gen = torch.Generator().manual_seed(11)
    lo, hi = math.log(16.0), math.log(float(args.max_prompt))
    lengths = [int(round(math.exp(lo + (hi - lo) * u))) for u in torch.rand(args.requests, generator=gen).tolist()]
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    sched = ContinuousScheduler(runner, max_concurrent=args.requests, chunk_size=2048, max_tokens_per_step=2048,
                                decode_headroom_blocks=8)
    # Warm-up: one short request end to end, so that kernels are built and loaded.
    sched.generate([Request(prompts[0][:64], SamplingParams(), max_tokens=4)])
    # ... and the decode steps of every batch size are captured, as the engine thread does before
    # it serves (ContinuousScheduler.start): a size met for the first time costs some 40 ms otherwise
    captured = runner.capture_decode_steps(args.requests)
    clocks = ClockSampler()
    clocks.start()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    handles = [sched.submit(Request(p, SamplingParams(), max_tokens=args.generate)) for p in prompts]
    step_ms, step_tokens, high_water, last = [], [], 0.0, t0
    while sched.step():
        now = time.perf_counter()
        step_ms.append(1000.0 * (now - last))
        step_tokens.append(sum(len(e.tokens) for e in sched.last_step_entries))
        high_water = max(high_water, sched.load_stats().kv_cache_usage)
        last = now
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    clock_summary = clocks.stop()
    results = [h.wait() for h in handles]
    sched.stop()
    runner.cache.check()
    generated = sum(len(r.tokens) for r in results)
    reasons: dict[str, int] = {}
    for r in results:
        reasons[r.finish_reason] = reasons.get(r.finish_reason, 0) + 1
    ordered = sorted(step_ms)
    decode_ms = sorted(ms for ms, n in zip(step_ms, step_tokens) if n <= args.requests)
    line = {
        "scenario": "long-mixed", "metric": "generated tokens a second, prefill included",
        "value": round(generated / wall, 1), "unit": "tokens/s", "wall_s": round(wall, 3),
        "prompt_tokens_per_s": round(sum(lengths) / wall, 1), "dtype": "bf16", "data": "synthetic",
        "config": {"model": model_name.replace(" ", "-") + " sizes, random weights", "layers": layers,
                   "layers_of_model": cfg["num_hidden_layers"], "requests": args.requests,
                   "prompt_tokens": sum(lengths), "longest_prompt": max(lengths), "shortest_prompt": min(lengths),
                   "generated_each": args.generate, "step_budget": 2048, "page_size": PAGE,
                   "pool_pages": num_blocks, "pool_gb": args.pool_gb},
        "steps": len(step_ms), "generated": generated, "finish_reasons": reasons,
        "step_ms": {"p50": round(ordered[len(ordered) // 2], 3), "p90": round(ordered[len(ordered) * 9 // 10], 3),
                    "max": round(ordered[-1], 3)},
        "decode_step_ms_p50": round(decode_ms[len(decode_ms) // 2], 3) if decode_ms else None,
        "pool_high_water": round(high_water, 4), "pool_in_use_after": runner.cache.usage(),
        "preemptions": sched.preemptions, "tokens_computed_in_vain": sched.wasted_tokens,
        "decode_graphs_captured_ahead": captured, "clocks": clock_summary,
    }
    return line


def reference_arm(args) -> int:
    """The unmodified reference (installed under baseline/_ref) on the same metric: its own
    ``LlamaForCausalLM`` with random bf16 weights at the same sizes, its ``BlockPool`` /
    ``PagedKVCache``, its ``ModelRunner.forward_step_packed`` with its decode CUDA graph and
    FlashInfer attention where this process can run them (its published configuration), and
    its ``sample_tokens``.  Nothing of this repository's engine is on that path."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    line = {"impl": "reference"}
    if not os.path.isdir(os.path.join(ref, "mini_infer")):
        line["unavailable"] = ("the reference is not installed under baseline/_ref (the stated pip command fails "
                               "offline: its build backend, hatchling, is not in the wheelhouse; it installs from "
                               "a copy whose build-system table names setuptools, sources unchanged)")
        print(json.dumps(line))
        return 0
    try:
        line.update(_reference_measure(args, ref))
    except Exception as e:  # noqa: BLE001  (any failure of the reference is reported, not raised)
        line = {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}".replace("\n", " ")}
    print(json.dumps(line))
    return 0


class _IdTokenizer:
    """Stands in for a text tokenizer where the reference's scheduler wants one: a prompt is its
    token ids written as decimal numbers."""

    eos_token_id = -1

    def encode(self, text):
        return [int(t) for t in text.split()]

    def decode(self, ids):
        return " ".join(str(int(i)) for i in ids)


def _reference_runner(ref: str, layers: int, num_blocks: int, prefill_graph: bool):
    """The reference's own model, pool and runner at the benchmark's sizes, random bf16 weights."""
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    if ref not in sys.path:
        sys.path.insert(0, ref)
    from types import SimpleNamespace

    import torch
    from mini_infer.cache.block_pool import BlockPool
    from mini_infer.cache.packed_attention import effective_attention_backend
    from mini_infer.engine.model_runner import ModelRunner
    from mini_infer.models.llama.llama import LlamaConfig, LlamaForCausalLM

    raw = dict(LLAMA_8B, num_hidden_layers=layers)
    cfg = LlamaConfig.from_hf(SimpleNamespace(**raw))
    torch.manual_seed(0)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device("cuda"):
            model = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(prev)
    model = model.to(device="cuda", dtype=torch.bfloat16).eval()
    with torch.no_grad():      # the engine's own arm uses N(0, 0.02) weights; values do not change the work
        for prm in model.parameters():
            if prm.dim() == 2:
                prm.normal_(0.0, 0.02)
    backend = "flashinfer" if effective_attention_backend("flashinfer", "cuda", None) == "flashinfer" else "flash_attn"
    pool = BlockPool(num_blocks=num_blocks, block_size=PAGE, num_layers=cfg.num_hidden_layers,
                     num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, dtype=torch.bfloat16,
                     device="cuda", attention_backend=backend)
    runner = ModelRunner(model=model, tokenizer=_IdTokenizer(), device="cuda", block_pool=pool)
    graphs = []
    if backend == "flashinfer":          # the reference's published configuration (its decode and prefill graphs)
        for name, enable in (("decode", runner.enable_decode_graph),
                             ("prefill", runner.enable_prefill_graph if prefill_graph else None)):
            if enable is None:
                continue
            try:
                enable()
                graphs.append(name)
            except (ValueError, AttributeError):
                pass
    return runner, cfg, backend, graphs


def _serving_numbers(run_together, single_requests: int, concurrency: int, out_tokens: int) -> dict:
    """The reference's published workload (``scripts/bench/modal_model_metrics.py:126-204``):
    warm-up, then ``single_requests`` requests one after the other (median time to the first
    token, median decode speed after it) and one batch of ``concurrency`` started together
    (tokens a second over the batch's wall time, median time to the first token)."""
    for index in (100, 101):
        run_together([index], 16)
    run_together(list(range(200, 200 + concurrency)), 16)
    single = [run_together([index], out_tokens)[0] for index in range(single_requests)]
    batch = run_together(list(range(10, 10 + concurrency)), out_tokens)
    wall = max(r["times"][-1] for r in batch) - min(r["submit"] for r in batch)
    total = sum(len(r["times"]) for r in batch)
    return {
        "single": {
            "ttft_ms": round(statistics.median((r["times"][0] - r["submit"]) * 1000 for r in single), 2),
            "decode_tok_s": round(statistics.median((len(r["times"]) - 1) / (r["times"][-1] - r["times"][0])
                                                    for r in single), 1),
            "requests": single_requests,
        },
        "batch": {
            "concurrency": concurrency, "throughput_tok_s": round(total / wall, 1),
            "ttft_p50_ms": round(statistics.median((r["times"][0] - r["submit"]) * 1000 for r in batch), 2),
            "mean_output_tokens": round(total / len(batch), 1),
        },
    }


SERVING_PROMPT, SERVING_OUTPUT, SERVING_SINGLE, SERVING_CONCURRENCY = 1024, 128, 5, 16


def _serving_prompt(index: int, vocab: int) -> list[int]:
    import torch

    gen = torch.Generator().manual_seed(5000 + index)
    return torch.randint(0, vocab, (SERVING_PROMPT,), generator=gen).tolist()


def serving_ours(args) -> dict:
    import torch

    from mini_infer_b200.engine import ContinuousScheduler, Request
    from mini_infer_b200.sampling import SamplingParams

    _, cfg, _ = SIZES[args.sizes]
    # 2048 pages of 16 tokens hold 16 requests of 1,152 tokens with room to spare (the reference's pool)
    runner = build_runner(cfg, args.layers, num_blocks=2048, max_requests=SERVING_CONCURRENCY)
    sched = ContinuousScheduler(runner, max_concurrent=SERVING_CONCURRENCY)
    sched.start()

    def run_together(indices, max_tokens):
        records = [{} for _ in indices]
        handles = []
        for rec, index in zip(records, indices):
            rec["submit"] = time.perf_counter()
            rec["times"] = []
            handles.append(sched.submit(Request(_serving_prompt(index, cfg["vocab_size"]), SamplingParams(), max_tokens),
                                        on_token=lambda tok, rec=rec: rec["times"].append(time.perf_counter())))
        for h in handles:
            h.wait(timeout=600)
        return records

    clocks = ClockSampler()
    clocks.start()
    try:
        numbers = _serving_numbers(run_together, SERVING_SINGLE, SERVING_CONCURRENCY, SERVING_OUTPUT)
    finally:
        sched.stop()
    torch.cuda.synchronize()
    numbers["clocks"] = clocks.stop()
    numbers["path"] = "paged cache, own kernels, captured decode steps, decode look-ahead"
    return numbers


def serving_reference(args, ref: str) -> dict:
    import threading

    runner, cfg, backend, graphs = _reference_runner(ref, args.layers, num_blocks=2048, prefill_graph=True)
    from mini_infer.engine.sampler import SamplingParams
    from mini_infer.scheduler import ContinuousScheduler, Request

    sched = ContinuousScheduler(runner, max_concurrent=SERVING_CONCURRENCY)
    sched.start()
    tok = _IdTokenizer()

    def one(index, max_tokens, rec):
        request = Request(prompt=tok.decode(_serving_prompt(index, cfg.vocab_size)),
                          sampling_params=SamplingParams(), max_tokens=max_tokens)
        rec["submit"] = time.perf_counter()
        rec["times"] = []
        handle = sched.submit(request)
        while True:
            step = handle.get_step(timeout=600)
            if step.failed:
                raise RuntimeError(f"request {index} failed")
            rec["times"].extend([time.perf_counter()] * step.num_tokens)
            if step.finish_reason is not None:
                break

    def run_together(indices, max_tokens):
        records = [{} for _ in indices]
        threads = [threading.Thread(target=one, args=(i, max_tokens, r)) for i, r in zip(indices, records)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if any(not r.get("times") for r in records):
            raise RuntimeError("a request of the reference arm produced nothing")
        return records

    clocks = ClockSampler()
    clocks.start()
    try:
        numbers = _serving_numbers(run_together, SERVING_SINGLE, SERVING_CONCURRENCY, SERVING_OUTPUT)
    finally:
        sched.stop()
    numbers["clocks"] = clocks.stop()
    numbers["path"] = f"paged, {backend} attention, graphs: {', '.join(graphs) or 'none'}"
    return numbers


def run_serving(args) -> int:
    model_name, cfg, _ = SIZES[args.sizes]
    line = {"scenario": "serving", "impl": args.impl,
            "metric": "reference-shaped serving: time to first token, single-request decode tok/s, tok/s of 16 together",
            "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (uniform token ids, no end-of-sequence id)",
            "config": {"model": model_name.replace(" ", "-") + " sizes, random weights", "layers": args.layers,
                       "layers_of_model": cfg["num_hidden_layers"], "prompt_tokens": SERVING_PROMPT,
                       "output_tokens": SERVING_OUTPUT, "single_requests": SERVING_SINGLE,
                       "concurrency": SERVING_CONCURRENCY, "page_size": PAGE, "pool_pages": 2048},
            "published_by_the_reference": {"single_decode_tok_s": 276.0, "batch_throughput_tok_s": 2668.0,
                                           "ttft_ms": 34.0, "where": "docs/benchmarks/2026-11-05-model-metrics.md:55"}}
    if args.impl == "reference":
        ref = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref, "mini_infer")):
            print(json.dumps({"impl": "reference", "scenario": "serving",
                              "unavailable": "the reference is not installed under baseline/_ref"}))
            return 0
        try:
            line.update(serving_reference(args, ref))
        except Exception as e:  # noqa: BLE001
            line = {"impl": "reference", "scenario": "serving",
                    "unavailable": f"{type(e).__name__}: {str(e)[:300]}".replace("\n", " ")}
    else:
        line.update(serving_ours(args))
    if "batch" in line:
        line["value"] = line["batch"]["throughput_tok_s"]
        # both schedulers run with their own defaults, as the reference's script runs its own
        line["config"]["prompt_portion"] = ("256 tokens per request and step (the reference's default chunk_size)"
                                            if args.impl == "reference" else
                                            "up to the step's 2048-token budget, oldest request first (this engine's default)")
    print(json.dumps(line))
    return 0


def _reference_measure(args, ref: str) -> dict:
    import threading

    import torch

    warmup = max(3, args.warmup)
    batch, steps, layers = args.batch, args.steps, args.layers
    tokens_cap = batch * (CONTEXT + 2 * (steps + warmup) + 128)
    runner, cfg, backend, graphs = _reference_runner(ref, layers, num_blocks=tokens_cap // PAGE + 8 * batch + 8,
                                                     prefill_graph=False)
    from mini_infer.cache.paged_kv_cache import PagedKVCache
    from mini_infer.engine.sampler import SamplingParams, sample_tokens
    from mini_infer.scheduler import ContinuousScheduler, Request

    graph = "decode" in graphs
    pool = runner.block_pool
    cache = PagedKVCache(pool)
    for _ in range(batch):
        cache.add_request_slot()
    gen = torch.Generator().manual_seed(3)
    chunk = 256                                     # the reference's default prompt portion
    prompts = [torch.randint(0, cfg.vocab_size, (CONTEXT,), generator=gen).tolist() for _ in range(batch)]
    for s0 in range(0, CONTEXT, chunk):             # every request brings one portion per step
        ids = [t for p in prompts for t in p[s0:s0 + chunk]]
        runner.forward_step_packed(cache, ids, [chunk * i for i in range(batch + 1)], cache.seq_lens_list(),
                                   last_rows_only=True)
    params = [SamplingParams()] * batch
    cu = list(range(batch + 1))

    def one(ids):
        logits = runner.forward_step_packed(cache, ids, cu, cache.seq_lens_list(), last_rows_only=True)
        return sample_tokens(logits[0].float(), params)

    ids = torch.randint(0, cfg.vocab_size, (batch,), generator=gen).tolist()
    clocks = ClockSampler()
    clocks.start()
    for _ in range(warmup):
        one(ids)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one(ids)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    cache.free()
    del cache
    # End to end through the reference's own scheduler (its engine thread, its sampling on the
    # device with ids read a step late): `batch` requests of CONTEXT prompt tokens are submitted
    # together; once every one of them has produced `warmup` tokens the clock runs until every
    # one has produced `steps` more.  Host token ids in (the prompts), sampled ids out per step.
    sched = ContinuousScheduler(runner, max_concurrent=batch)
    sched.start()
    tok = _IdTokenizer()
    want = warmup + steps
    stamps: list[list[float]] = [[] for _ in range(batch)]

    def follow(i):
        handle = sched.submit(Request(prompt=tok.decode(prompts[i]), sampling_params=SamplingParams(),
                                      max_tokens=want + 4))
        while True:
            step = handle.get_step(timeout=600)
            if step.failed:
                raise RuntimeError("a request of the reference arm failed")
            stamps[i].extend([time.perf_counter()] * step.num_tokens)
            if step.finish_reason is not None:
                break

    threads = [threading.Thread(target=follow, args=(i,)) for i in range(batch)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    sched.stop()
    if any(len(st) < want for st in stamps):
        raise RuntimeError("the reference's scheduler produced fewer tokens than asked for")
    t_a = max(st[warmup - 1] for st in stamps)
    t_b = max(st[want - 1] for st in stamps)
    dt = t_b - t_a
    value = batch * 1000.0 / ms
    return {
        "metric": "decode tok/s @ batch 8, 2048-token context (Llama 3.1 8B layer sizes)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / BASELINE_DECODE_TOK_S, 3), "dtype": "bf16", "data": "synthetic",
        "config": {"model": "Llama-3.1-8B sizes, random weights", "layers": layers,
                   "layers_of_model": LLAMA_8B["num_hidden_layers"], "global_batch": batch, "seq_len": CONTEXT,
                   "page_size": PAGE, "attention_backend": backend, "cuda_graph": graph,
                   "parallelism": "single GPU", "l2": "inputs (weights) larger than L2, no flush",
                   "e2e_path": "the reference's ContinuousScheduler (engine thread, asynchronous sampling)"},
        "e2e": {"value": round(batch * steps / dt, 2), "unit": "tokens/s", "ms_per_step": round(1000.0 * dt / steps, 3),
                "h2d_bytes_per_step": 8 * batch, "d2h_bytes_per_step": 8 * batch},
        "clocks": clocks.stop(),
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sizes", default="8b", choices=sorted(SIZES), help="layer sizes of which model")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has (sizes unchanged), for small memory")
    ap.add_argument("--context", type=int, default=CONTEXT, help="tokens each request holds when decoding starts")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 and e2e measurements")
    ap.add_argument("--scenario", default="decode", choices=["decode", "long-mixed", "serving"],
                    help="decode: the contract line; long-mixed: many requests of very different lengths "
                         "through the scheduler (a line of its own); serving: the reference's published "
                         "workload, 1024 tokens in and 128 out, single requests and 16 together (a line of its own)")
    ap.add_argument("--requests", type=int, default=64, help="long-mixed: requests started together")
    ap.add_argument("--max-prompt", type=int, default=32768, help="long-mixed: longest prompt")
    ap.add_argument("--generate", type=int, default=256, help="long-mixed: tokens generated per request")
    ap.add_argument("--pool-gb", type=float, default=48.0, help="long-mixed: size of the key/value pool")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    model_name, cfg, default_layers = SIZES[args.sizes]
    if args.layers is None:
        args.layers = default_layers
    if args.scenario == "serving":
        if args.impl == "reference" and args.sizes != "8b":
            print(json.dumps({"impl": "reference", "scenario": "serving",
                              "unavailable": "the reference arm runs the 8B sizes only"}))
            return 0
        return run_serving(args)
    if args.impl == "reference":
        if args.sizes != "8b" or args.scenario != "decode" or args.context != CONTEXT:
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm measures the contract's "
                              "configuration only (8B sizes, decode, 2048-token context)"}))
            return 0
        return reference_arm(args)
    if args.scenario == "long-mixed":
        return run_long_mixed(args)
    warmup = max(3, args.warmup)

    import torch

    from mini_infer_b200.csrc import build as kernel_build

    layers, batch, context = args.layers, args.batch, args.context
    peaks = load_peaks()
    point_batches = () if args.skip_points else POINTS[args.sizes]
    max_batch = max((batch, *point_batches))
    tokens_cap = max_batch * (context + args.steps + warmup + 2 * batch + 64)
    runner = build_runner(cfg, layers, num_blocks=tokens_cap // PAGE + 8, max_requests=max_batch)

    clocks = ClockSampler()
    clocks.start()
    ms, launches = time_decode(runner, batch, context, args.steps, warmup)
    points, e2e, prefill = {}, None, None
    prefill_ms = time_prefill(runner, PREFILL_TOKENS, repeats=3, warmup=2)
    if not args.skip_points:
        for b in point_batches:
            pms, _ = time_decode(runner, b, context, args.steps, warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
        e2e = time_e2e(runner, batch, context, args.steps, warmup)
    clock_summary = clocks.stop()

    value = batch * 1000.0 / ms
    mean_ctx = context + warmup + args.steps / 2.0
    achieved = decode_bytes(cfg, layers, batch, mean_ctx) / (ms * 1e-3) / 1e9
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    line = {
        "metric": f"decode tok/s @ batch {batch}, {context}-token context ({model_name} layer sizes)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / BASELINE_DECODE_TOK_S, 3) if args.sizes == "8b" else None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": model_name.replace(" ", "-") + " sizes, random weights", "layers": layers,
            "layers_of_model": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": batch, "seq_len": context, "context_cap": max(4096, 2 * context), "page_size": PAGE,
            "prefill_tokens": PREFILL_TOKENS, "kv_dtype": "bf16", "parallelism": "single GPU",
            "l2": "inputs (weights) larger than L2, no flush", "peaks": peaks["source"],
        },
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "gpu_launches": launches,
        "clocks": clock_summary,
        "kernel_libraries": sorted(os.path.basename(kernel_build.library_path(n)) for n in kernel_build._loaded),
    }
    if e2e is not None:
        line["e2e"] = {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
