"""The scheduler's decisions, with a scripted step function over a real cache manager
(no GPU): admission, the token budget, portions, finishing, and what happens when pages
run out.  The fake logits name the request and position they came from, so the tests see
which row every request read (the reference tests its scheduler the same way,
tests/unit/scheduler/test_scheduler_variable_tokens.py:44-110)."""

from types import SimpleNamespace

import pytest

from mini_infer_b200.cache import CacheManager
from mini_infer_b200.engine.scheduler import ContinuousScheduler, Request, RequestState
from mini_infer_b200.parts import KVNeed
from mini_infer_b200.sampling import SamplingParams

VOCAB = 1000


def token_for(rid, position):
    return (rid * 131 + position * 7 + 3) % (VOCAB - 1) + 1      # never 0 (0 is the end id in one test)


class FakeRunner:
    """Keeps the fed tokens per request and answers each wanted row with (rid, position)."""

    def __init__(self, num_pages, page_size=4, max_requests=8, max_positions=None):
        needs = [SimpleNamespace(index=0, kv=KVNeed(1, 16), state=None)]
        self.cache = CacheManager(needs, page_size=page_size, num_pages=num_pages, max_requests=max_requests)
        self.device = None
        self.max_positions = max_positions
        self.fed = {}            # rid -> tokens currently in the cache
        self.log = []            # per step: [(rid, n_tokens, start_position, wants)]

    def step(self, entries):
        plan = self.cache.plan_append([(e.rid, len(e.tokens)) for e in entries])
        rows, rec = [], []
        for e, start in zip(entries, plan.start):
            if start == 0:
                self.fed[e.rid] = []
            assert len(self.fed[e.rid]) == start
            self.fed[e.rid].extend(e.tokens)
            rec.append((e.rid, len(e.tokens), start, list(e.want)))
            for w in e.want:
                rows.append((e.rid, start + w))
        self.log.append(rec)
        self.cache.check()
        return SimpleNamespace(logits=rows, rows=rows)


class FakeSampler:
    def __init__(self, eos_at=None):
        self.eos_at = eos_at or {}
        self.calls = []

    def sample(self, logits, params, seeds, draw_index):
        self.calls.append((list(logits), list(draw_index)))
        out = []
        for (rid, pos), n in zip(logits, draw_index):
            out.append(0 if self.eos_at.get(rid) == n else token_for(rid, pos))
        return out


def make(num_pages=64, **kw):
    runner = FakeRunner(num_pages, page_size=kw.pop("page_size", 4), max_requests=kw.pop("max_requests", 8),
                        max_positions=kw.pop("max_positions", None))
    sampler = kw.pop("sampler", FakeSampler())
    sched = ContinuousScheduler(runner, sampler=sampler, **kw)
    return runner, sched


def expected_tokens(rid, prompt_len, n):
    return [token_for(rid, prompt_len - 1 + i) for i in range(n)]


def prompt(n, base=100):
    return [(base + i) % VOCAB for i in range(n)]


def test_generates_and_frees_everything():
    runner, sched = make(max_tokens_per_step=64, chunk_size=64)
    results = sched.generate([Request(prompt(n), SamplingParams(), 5) for n in (1, 17, 48)])
    for rid, (res, n) in enumerate(zip(results, (1, 17, 48))):
        assert res.finish_reason == "length" and res.prompt_tokens == n
        assert res.tokens == expected_tokens(rid, n, 5)
    assert runner.cache.num_requests == 0 and runner.cache.num_free_pages() == 64
    # what was fed is the prompt followed by the generated tokens but the last
    for rid, n in enumerate((1, 17, 48)):
        assert runner.fed[rid] == prompt(n) + results[rid].tokens[:-1]


def test_without_a_chunk_size_prompts_are_fed_oldest_first_and_whole_where_they_fit():
    runner, sched = make(max_tokens_per_step=64, decode_headroom_blocks=0)
    sched.generate([Request(prompt(40), max_tokens=1), Request(prompt(40), max_tokens=1),
                    Request(prompt(40), max_tokens=1)])
    # step 0: the first prompt whole, the second gets what the budget leaves; step 1: its rest, then the third
    assert [(r, n) for r, n, _, _ in runner.log[0]] == [(0, 40), (1, 24)]
    assert [(r, n) for r, n, _, _ in runner.log[1]] == [(1, 16), (2, 40)]
    assert len(runner.log) == 2


def test_token_budget_decoders_first_then_portions_in_order():
    runner, sched = make(max_tokens_per_step=10, chunk_size=6, decode_headroom_blocks=0)
    sched.generate([Request(prompt(3), max_tokens=30), Request(prompt(20), max_tokens=2),
                    Request(prompt(9), max_tokens=2)])
    for rec in runner.log:
        assert sum(n for _, n, _, _ in rec) <= 10
        assert all(n <= 6 for _, n, _, _ in rec)
        kinds = ["d" if (n == 1 and start > 0 and start >= {0: 3, 1: 20, 2: 9}[rid]) else "p"
                 for rid, n, start, _ in rec]
        assert kinds == sorted(kinds), "decoding tokens come before prompt portions"
    # step 0: request 0 whole (3), request 1 gets min(chunk, budget left) = 6, request 2 the last token of budget
    assert [(r, n) for r, n, _, _ in runner.log[0]] == [(0, 3), (1, 6), (2, 1)]
    # step 1: request 0 decodes (1), then 1 gets 6, then 2 is cut to what is left (3)
    assert [(r, n) for r, n, _, _ in runner.log[1]] == [(0, 1), (1, 6), (2, 3)]
    # logits are wanted only where a prompt ends or a token is decoded
    for rec in runner.log:
        for rid, n, start, want in rec:
            ends_prompt = start + n == {0: 3, 1: 20, 2: 9}[rid]
            decoding = start >= {0: 3, 1: 20, 2: 9}[rid]
            assert want == ([n - 1] if (ends_prompt or decoding) else [])


def test_portions_can_be_as_small_as_one_token():
    runner, sched = make(max_tokens_per_step=3, chunk_size=2)
    res = sched.generate([Request(prompt(7), max_tokens=3), Request(prompt(5), max_tokens=3)])
    assert [r.tokens for r in res] == [expected_tokens(0, 7, 3), expected_tokens(1, 5, 3)]
    sizes = {n for rec in runner.log for _, n, _, _ in rec}
    assert sizes == {1, 2}


def test_admission_is_fifo_and_bounded():
    runner, sched = make(num_pages=64, max_concurrent=2, max_tokens_per_step=64)
    handles = [sched.submit(Request(prompt(4), max_tokens=3)) for _ in range(5)]
    sched.step()
    assert sched.load_stats().num_running == 2 and sched.load_stats().num_waiting == 3
    assert {rid for rid, *_ in runner.log[0]} == {0, 1}
    sched.run_until_done()
    first_seen = {}
    for i, rec in enumerate(runner.log):
        for rid, *_ in rec:
            first_seen.setdefault(rid, i)
    assert [first_seen[r] for r in range(5)] == sorted(first_seen[r] for r in range(5))
    assert all(h.wait().finish_reason == "length" for h in handles)
    stats = sched.load_stats()
    assert (stats.num_running, stats.num_waiting, stats.kv_cache_usage) == (0, 0, 0.0)
    assert (stats.block_size, stats.num_blocks) == (4, 64)


def test_admission_waits_for_pages_and_keeps_headroom():
    runner, sched = make(num_pages=10, max_tokens_per_step=64, chunk_size=64, decode_headroom_blocks=2)
    sched.submit(Request(prompt(20), max_tokens=4))       # 6 pages with its first decoded token
    sched.submit(Request(prompt(12), max_tokens=4))       # 4 pages + 2 headroom: must wait
    sched.step()
    assert sched.load_stats().num_running == 1 and sched.load_stats().num_waiting == 1
    sched.run_until_done()
    assert runner.cache.num_free_pages() == 10


def test_finish_reasons():
    sampler = FakeSampler(eos_at={0: 2})
    runner, sched = make(sampler=sampler, eos_token_ids=[0])
    a = sched.submit(Request(prompt(5), max_tokens=10))
    b = sched.submit(Request([], max_tokens=10))
    c = sched.submit(Request(prompt(500), max_tokens=10))          # 126 pages > pool of 64
    sched.run_until_done()
    ra, rb, rc = a.wait(), b.wait(), c.wait()
    assert ra.finish_reason == "stop" and ra.tokens == expected_tokens(0, 5, 2)   # the end id is not emitted
    assert rb.finish_reason == "stop" and rb.tokens == []
    assert rc.finish_reason == "cancelled" and rc.tokens == []
    with pytest.raises(ValueError):
        sched.submit(Request(prompt(3), max_tokens=0))


def test_last_position_of_the_model_ends_a_request():
    runner, sched = make(max_positions=12)
    res = sched.run(Request(prompt(9), max_tokens=50))
    assert res.finish_reason == "length" and len(res.tokens) == 4     # tokens at positions 9, 10, 11 fed; 12th position never
    assert max(start + n for rec in runner.log for _, n, start, _ in rec) <= 12
    assert sched.run(Request(prompt(12), max_tokens=5)).finish_reason == "cancelled"


def test_when_pages_run_out_portions_shrink_then_the_youngest_is_recomputed():
    # 8 pages of 4 tokens.  Two requests decode until the pool is full; then the youngest is
    # preempted, recomputed later, and still produces exactly the tokens it would have.
    runner, sched = make(num_pages=8, max_tokens_per_step=64, chunk_size=64, decode_headroom_blocks=0)
    res = sched.generate([Request(prompt(10), max_tokens=14), Request(prompt(9), max_tokens=14)])
    assert sched.preemptions >= 1
    assert res[0].tokens == expected_tokens(0, 10, 14) and res[0].finish_reason == "length"
    assert res[1].tokens == expected_tokens(1, 9, 14) and res[1].finish_reason == "length"
    assert runner.cache.num_free_pages() == 8 and runner.cache.num_requests == 0
    # the preempted request was fed its prompt plus what it had generated, from position 0
    restarts = [rec for rec in runner.log for rid, n, start, _ in rec if rid == 1 and start == 0]
    assert len(restarts) >= 2
    # no token was emitted twice: draw indices per request are 0, 1, 2, ... without repeats
    draws = {}
    for rows, idx in sched.sampler.calls:
        for (rid, _), n in zip(rows, idx):
            draws.setdefault(rid, []).append(n)
    assert draws[0] == list(range(14)) and draws[1] == list(range(14))


def test_prompt_portions_shrink_to_the_pages_that_are_left():
    runner, sched = make(num_pages=6, max_tokens_per_step=64, chunk_size=64, decode_headroom_blocks=0)
    a = sched.submit(Request(prompt(14), max_tokens=3))
    sched.step()                                    # a: 14 tokens, 4 pages
    b = sched.submit(Request(prompt(7), max_tokens=2))
    sched.run_until_done()
    assert a.wait().tokens == expected_tokens(0, 14, 3)
    assert b.wait().tokens == expected_tokens(1, 7, 2)
    assert runner.cache.num_free_pages() == 6


def test_a_request_that_cannot_fit_alone_is_cancelled():
    runner, sched = make(num_pages=3, max_tokens_per_step=64, chunk_size=64, decode_headroom_blocks=0)
    res = sched.run(Request(prompt(10), max_tokens=20))       # needs a 4th page at token 13
    assert res.finish_reason == "cancelled" and res.tokens == expected_tokens(0, 10, len(res.tokens))
    assert runner.cache.num_free_pages() == 3


def test_cancel_and_engine_thread():
    runner, sched = make()
    h = sched.submit(Request(prompt(6), max_tokens=1000))
    sched.step()
    h.cancel()
    assert h.wait().finish_reason == "cancelled" and runner.cache.num_free_pages() == 64
    sched.start()
    try:
        out = sched.submit(Request(prompt(5), max_tokens=4)).wait(timeout=20)
        assert out.tokens == expected_tokens(1, 5, 4)
    finally:
        sched.stop()


def test_trace_out(tmp_path):
    import json

    path = tmp_path / "trace.json"
    runner, sched = make(trace_out=str(path), max_tokens_per_step=8, chunk_size=8)
    sched.generate([Request(prompt(12), max_tokens=2), Request(prompt(2), max_tokens=4)])
    sched.stop()
    events = json.loads(path.read_text())["traceEvents"]
    assert len(events) == len(runner.log)
    assert {e["args"]["phase"] for e in events} <= {"prefill", "decode", "mixed"}
    assert events[0]["args"]["total_q"] == 8 and events[0]["args"]["B"] == 1


# ----------------------------------------------------------------------------- decode look-ahead


class FeedbackRunner(FakeRunner):
    """A runner that takes the next tokens from a tensor (the sampler's output), as the real
    one does on the device."""

    device_token_feedback = True

    def step(self, entries, device_tokens=None):
        if device_tokens is not None:
            assert all(len(e.tokens) == 1 for e in entries)
            entries = [SimpleNamespace(rid=e.rid, tokens=[int(t)], want=e.want)
                       for e, t in zip(entries, device_tokens.tolist())]
        return super().step(entries)


class TensorSampler(FakeSampler):
    def sample(self, logits, params, seeds, draw_index):
        import torch

        return torch.tensor(super().sample(logits, params, seeds, draw_index), dtype=torch.int32)


def make_lookahead(num_pages=64, eos_at=None, **kw):
    runner = FeedbackRunner(num_pages, page_size=4, max_requests=8)
    sched = ContinuousScheduler(runner, sampler=TensorSampler(eos_at), **kw)
    assert sched.lookahead
    return runner, sched


def test_lookahead_gives_the_same_tokens_and_frees_everything():
    requests = [Request(prompt(n), SamplingParams(), m) for n, m in ((5, 9), (17, 4), (30, 12))]
    _, plain = make(max_tokens_per_step=64, chunk_size=64)
    want = [r.tokens for r in plain.generate(requests)]
    runner, sched = make_lookahead(max_tokens_per_step=64, chunk_size=64)
    got = sched.generate(requests)
    assert [r.tokens for r in got] == want
    assert all(r.finish_reason == "length" for r in got)
    assert sched.wasted_tokens == 0, "a length is known before the step is launched"
    assert runner.cache.num_requests == 0 and runner.cache.num_free_pages() == 64
    for rid, (n, _) in enumerate(((5, 9), (17, 4), (30, 12))):
        assert runner.fed[rid] == prompt(n) + got[rid].tokens[:-1]
    # while all three decode, two steps are in flight per call: fewer calls than steps is not
    # observable here, but every decode step after the first was fed from the sampler's tensor
    assert sched.steps == plain.steps


def test_lookahead_stop_token_costs_one_token_and_its_pages_come_back():
    eos = {1: 3}          # request 1 samples the end id as its fourth token
    requests = [Request(prompt(6), SamplingParams(), 10), Request(prompt(9), SamplingParams(), 10)]
    _, plain = make(max_tokens_per_step=64, chunk_size=64, eos_token_ids=[0], sampler=FakeSampler(eos))
    want = plain.generate(requests)
    runner, sched = make_lookahead(eos_at=eos, max_tokens_per_step=64, chunk_size=64, eos_token_ids=[0])
    got = sched.generate(requests)
    assert [r.tokens for r in got] == [r.tokens for r in want]
    assert [r.finish_reason for r in got] == ["length", "stop"]
    assert sched.wasted_tokens == 1
    assert runner.cache.num_requests == 0 and runner.cache.num_free_pages() == 64


def test_lookahead_drains_when_a_request_arrives():
    runner, sched = make_lookahead(max_tokens_per_step=64, chunk_size=64)
    first = sched.submit(Request(prompt(7), SamplingParams(), 12))
    for _ in range(4):
        sched.step()
    assert sched._inflight is not None, "a lone decoding request runs one step ahead"
    second = sched.submit(Request(prompt(11, base=300), SamplingParams(), 5))
    sched.run_until_done()
    assert first.wait().tokens == expected_tokens(0, 7, 12)
    assert second.wait().tokens == expected_tokens(1, 11, 5)
    assert runner.cache.num_requests == 0 and runner.cache.num_free_pages() == 64


def test_lookahead_cancel_while_a_step_is_ahead():
    runner, sched = make_lookahead(max_tokens_per_step=64, chunk_size=64)
    h = sched.submit(Request(prompt(7), SamplingParams(), 50))
    other = sched.submit(Request(prompt(3, base=500), SamplingParams(), 8))
    for _ in range(3):
        sched.step()
    h.cancel()
    sched.run_until_done()
    assert h.wait().finish_reason == "cancelled"
    assert other.wait().tokens == expected_tokens(1, 3, 8)
    assert runner.cache.num_requests == 0 and runner.cache.num_free_pages() == 64


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_lookahead_random_arrivals_match_the_plain_scheduler(seed):
    """Requests of random lengths arrive at random moments into a pool so small that some are
    preempted; some end on a stop token; with and without decode look-ahead every request gets
    the same tokens and the same reason to finish, and every page comes back."""
    import random

    rng = random.Random(seed)
    n = rng.randint(3, 7)
    specs = [(rng.randint(1, 40), rng.randint(1, 25)) for _ in range(n)]          # (prompt length, max tokens)
    arrive = sorted(rng.randint(0, 30) for _ in range(n))                        # step at which each is submitted
    eos = {rid: rng.randint(0, m - 1) for rid, (_, m) in enumerate(specs) if rng.random() < 0.4}
    pages = rng.randint(14, 28)

    def run(lookahead):
        runner = FeedbackRunner(pages, page_size=4, max_requests=4)
        sched = ContinuousScheduler(runner, sampler=TensorSampler(dict(eos)), lookahead=lookahead, eos_token_ids=[0],
                                    max_concurrent=4, chunk_size=16, max_tokens_per_step=24, decode_headroom_blocks=0)
        handles, step, nxt = [], 0, 0
        while nxt < n or any(not h.finished for h in handles):
            while nxt < n and arrive[nxt] <= step:
                p, m = specs[nxt]
                handles.append(sched.submit(Request(prompt(p, base=37 * nxt), SamplingParams(), m)))
                nxt += 1
            sched.step()
            step += 1
            assert step < 2000, "the scheduler does not finish"
        sched.run_until_done()
        runner.cache.check()
        assert runner.cache.num_requests == 0 and runner.cache.num_free_pages() == pages
        return [(h.wait().tokens, h.wait().finish_reason) for h in handles], sched

    plain, _ = run(False)
    ahead, sched = run(True)
    assert ahead == plain
    assert sched.wasted_tokens <= len(eos)


def test_a_kernel_that_gave_up_waiting_cancels_the_step_and_raises():
    """The runner's health word is read with every step's tokens.  When it is set the tokens of
    that step are thrown away, its requests end as cancelled with their pages back, the runner
    is reset, and the error reaches whoever drives the engine; afterwards the engine works."""
    import torch

    from mini_infer_b200.engine.scheduler import EngineFaultError

    runner, sched = make(max_tokens_per_step=64, chunk_size=64)
    word = torch.zeros(1, dtype=torch.int32)
    resets = []
    runner.health_word = lambda: word
    runner.reset_health = lambda: (resets.append(True), word.zero_())
    handles = [sched.submit(Request(prompt(n), SamplingParams(), 6)) for n in (5, 9)]
    assert sched.step() and sched.step()
    emitted_before = [len(h._rr.generated) for h in handles]
    word.fill_(1)                                  # "a wait gave up" during the next step
    with pytest.raises(EngineFaultError, match="gave up"):
        sched.step()
    assert resets == [True] and int(word[0]) == 0
    assert all(h.finished and h.wait().finish_reason == "cancelled" for h in handles)
    assert [len(h.wait().tokens) for h in handles] == emitted_before      # nothing from the bad step
    assert runner.cache.num_requests == 0 and runner.cache.num_free_pages() == 64
    runner.cache.check()
    res = sched.generate([Request(prompt(4), SamplingParams(), 3)])[0]
    assert res.finish_reason == "length" and len(res.tokens) == 3


def test_streaming_callback_may_call_back_into_the_scheduler():
    """Callbacks run outside the scheduler's lock: one that cancels its own request, asks for
    the load and submits another request does not deadlock."""
    runner, sched = make(max_tokens_per_step=64, chunk_size=64)
    seen, later = [], []

    def on_token(tok):
        seen.append(tok)
        assert sched.load_stats().block_size == 4
        if len(seen) == 3:
            later.append(sched.submit(Request(prompt(2), SamplingParams(), 2)))
            handle.cancel()

    handle = sched.submit(Request(prompt(7), SamplingParams(), 50), on_token=on_token)
    sched.run_until_done()
    res = handle.wait()
    assert res.finish_reason == "cancelled" and res.tokens == seen and len(seen) == 3
    assert later[0].wait().finish_reason == "length"
    assert runner.cache.num_requests == 0
