"""The engine against the plain implementation under every way of cutting the work,
in 32-bit and in bfloat16, for two tiny configurations."""

import numpy as np
import pytest
import torch

import trace_util as T
from tiny_configs import PAGE_SIZE, TINY, load_state, prompt_ids

pytestmark = pytest.mark.gpu

# tolerances: trace_util.tolerance (float32 1e-4 of max(1, |logit|); bfloat16 1e-2 of |logit|)

LENGTHS = {
    "A": [17, 33, 64, 5, 70, 90],        # prompts 1/17/48 plus 16 decoded, and three more
    "B": [25, 31, 87, 154, 224, 3],      # prompts 1/7/63/130/200 plus 24 decoded, and one more
    "C": [40, 130, 65, 7, 200, 96],      # ends inside a page, inside a 64-key chunk, on a chunk's edge
}


def requests_for(which):
    return {f"r{i}": prompt_ids(which, n, salt=i) for i, n in enumerate(LENGTHS[which])}


@pytest.fixture(scope="module")
def plain(model_dirs):
    out = {}
    for which in ("A", "B", "C"):
        state = load_state(model_dirs[which])
        out[which] = T.plain_logits(state, TINY[which], requests_for(which))
    return out


def make_runner(model_dir, which, dtype, steps):
    from mini_infer_b200.engine import ModelRunner

    ps = PAGE_SIZE[which]
    runner = ModelRunner.from_pretrained(model_dir, dtype=dtype, block_size=ps,
                                         num_blocks=T.max_tokens_needed(steps) // ps, max_requests=4)
    for st in runner.cache.storage:
        st.fill_(float("nan"))       # a slot that was never written must never be read
    return runner


CUTTINGS = {
    "whole": T.cut_whole,
    "last_decoded": T.cut_last_decoded,
    "portions": T.cut_portions,
    "mixed": T.cut_mixed,
}


@pytest.mark.parametrize("cutting", list(CUTTINGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_replay_matches_plain(which, dtype, cutting, model_dirs, plain):
    requests = requests_for(which)
    steps = CUTTINGS[cutting](requests)
    if cutting == "mixed":
        assert max(len(s["entries"]) for s in steps) == 4
        assert any(len(e["tokens"]) > 1 for s in steps for e in s["entries"] if len(s["entries"]) > 1)
    runner = make_runner(model_dirs[which], which, dtype, steps)
    got = T.collect(steps, T.replay_in_process(runner, steps), TINY[which]["vocab_size"])
    runner.cache.check()
    assert runner.cache.num_requests == 0
    assert runner.cache.num_free_pages() == runner.cache.pools[0].num_pages
    if dtype == "bfloat16":
        from mini_infer_b200.csrc import ops
        assert ops.attention_wait_status() == 0
        if which == "C":     # the sizes of C are the ones the tcgen05 kernels take
            cfg = TINY[which]
            assert ops.prefill_tc_supported(cfg["num_attention_heads"], cfg["num_key_value_heads"],
                                            cfg["head_dim"], PAGE_SIZE[which])
            assert ops.attention_tc_status() == 0 and ops.gemm_tma_status() == 0
    want = plain[which]
    scale = max(float(np.abs(want[r]).max()) for r in want)
    for rid in requests:
        assert got[rid].shape == want[rid].shape
        assert np.isfinite(got[rid]).all(), f"{rid}: non-finite logits"
        bad = T.first_bad(got[rid], want[rid], T.tolerance(dtype, scale))
        assert bad is None, (
            f"{which}/{dtype}/{cutting}: request {rid} first differs at position {bad} "
            f"(page size {PAGE_SIZE[which]}), |diff| = {np.abs(got[rid][bad] - want[rid][bad]).max():.3e}"
        )


@pytest.mark.parametrize("which", ["A", "B"])
def test_fp32_cuttings_agree_closely(which, model_dirs):
    """In 32-bit every cutting gives the same logits bit for bit: every sum in the fp32
    kernels runs in an order that depends on the position alone."""
    requests = requests_for(which)
    results = {}
    for name, cut in CUTTINGS.items():
        steps = cut(requests)
        runner = make_runner(model_dirs[which], which, "float32", steps)
        results[name] = T.collect(steps, T.replay_in_process(runner, steps), TINY[which]["vocab_size"])
    for name in ("last_decoded", "portions", "mixed"):
        err, scale = T.max_err(results[name], results["whole"])
        assert err == 0.0, f"{name} vs whole: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, model_dirs, plain, tmp_path):
    """The program itself, as a user runs it: mixed cutting with pages used again."""
    which = "A"
    requests = requests_for(which)
    steps = T.cut_mixed(requests)
    per_step = T.replay_program(model_dirs[which], dtype, steps, str(tmp_path / "out"),
                                block_size=PAGE_SIZE[which])
    got = T.collect(steps, per_step, TINY[which]["vocab_size"])
    err, scale = T.max_err(got, plain[which])
    assert err <= T.tolerance(dtype, scale)


def test_first_tokens_and_long_decoding(model_dirs, plain):
    """The first tokens of a sequence (positions 0, 1, 2 alone in their steps) and a long
    run of single-token steps crossing many page edges."""
    which = "B"
    toks = prompt_ids(which, 224, salt=4)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []}
             for i, t in enumerate(toks)]
    steps[-1]["end"] = ["x"]
    for dtype in ("float32", "bfloat16"):
        runner = make_runner(model_dirs[which], which, dtype, steps)
        got = T.collect(steps, T.replay_in_process(runner, steps), TINY[which]["vocab_size"])["x"]
        want = plain[which]["r4"]
        bad = T.first_bad(got, want, T.tolerance(dtype, float(np.abs(want).max())))
        assert bad is None, f"{dtype}: token-by-token decoding first differs at position {bad}"


def test_out_of_pages_changes_nothing(model_dirs):
    from mini_infer_b200.cache import OutOfPages
    from mini_infer_b200.engine import ModelRunner, StepEntry

    runner = ModelRunner.from_pretrained(model_dirs["A"], dtype="float32", block_size=16, num_blocks=3,
                                         max_requests=2)
    runner.add_request("a")
    runner.add_request("b")
    runner.step([StepEntry("a", prompt_ids("A", 30), [29])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("a", [1], [0]), StepEntry("b", prompt_ids("A", 40), [])])
    assert runner.cache.length("a") == 30 and runner.cache.length("b") == 0
    assert runner.cache.num_free_pages() == 1
    runner.cache.check()


@pytest.mark.parametrize("which,dtype", [("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16")])
def test_captured_decode_steps_match_plain(which, dtype, model_dirs, plain):
    """With cuda_graph on, single-token steps replay captured CUDA graphs (one per batch
    size); prompt portions and mixed steps still run kernel by kernel.
    Inside a captured step the kernels overlap through programmatic dependent launch (with
    configuration C: the tcgen05 product and decode attention that work ahead of their inputs)."""
    from mini_infer_b200.engine import ModelRunner

    requests = requests_for(which)
    steps = T.cut_mixed(requests, n_decode=40)
    ps = PAGE_SIZE[which]
    runner = ModelRunner.from_pretrained(model_dirs[which], dtype=dtype, block_size=ps,
                                         num_blocks=T.max_tokens_needed(steps) // ps, max_requests=4,
                                         cuda_graph=True)
    got = T.collect(steps, T.replay_in_process(runner, steps), TINY[which]["vocab_size"])
    assert sum(slot.replays for slot in runner.stepper._graphs.values()) >= 20
    assert len(runner.stepper._graphs) >= 2          # several batch sizes were captured
    want = plain[which]
    scale = max(float(np.abs(want[r]).max()) for r in want)
    for rid in requests:
        bad = T.first_bad(got[rid], want[rid], T.tolerance(dtype, scale))
        assert bad is None, f"{dtype}: request {rid} first differs at position {bad}"
    runner.cache.check()


def test_one_long_request_among_short_ones(model_dirs):
    """Decode steps of a batch whose longest request (1,540 tokens) is many times the others
    (40 and 200): the decode kernel spreads the long request's keys over many blocks while the
    short ones share one; eight captured steps (one graph: the lengths are read on the device)
    against the plain implementation."""
    from mini_infer_b200.engine import ModelRunner

    which, dtype, n_decode = "C", "bfloat16", 8
    requests = {"long": prompt_ids(which, 1540, salt=7), "short": prompt_ids(which, 40, salt=8),
                "mid": prompt_ids(which, 200, salt=9)}
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:-n_decode], "want": []}], "end": []})
    for i in range(n_decode):
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": rid, "tokens": [toks[len(toks) - n_decode + i]], "want": [0]}
                                  for rid, toks in requests.items()]})
    steps[-1]["end"] = list(requests)
    ps = PAGE_SIZE[which]
    runner = ModelRunner.from_pretrained(model_dirs[which], dtype=dtype, block_size=ps,
                                         num_blocks=T.max_tokens_needed(steps) // ps, max_requests=4,
                                         cuda_graph=True)
    for st in runner.cache.storage:
        st.fill_(float("nan"))
    got = T.collect(steps, T.replay_in_process(runner, steps), TINY[which]["vocab_size"])
    assert list(runner.stepper._graphs) == [(3,)] and runner.stepper._graphs[(3,)].replays == n_decode - 1
    want = T.plain_logits(load_state(model_dirs[which]), TINY[which], requests)
    scale = max(float(np.abs(want[r]).max()) for r in want)
    for rid in requests:
        bad = T.first_bad(got[rid], want[rid][-n_decode:], T.tolerance(dtype, scale))
        assert bad is None, f"request {rid} first differs at decoded token {bad}"
    runner.cache.check()
