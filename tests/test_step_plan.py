"""The host side of a step's plan, without a GPU: what is laid out for the device, that it
does not grow with the context, and that it is cheap."""

import time
from types import SimpleNamespace

import torch

from mini_infer_b200.cache import CacheManager
from mini_infer_b200.engine.step import StepEntry, StepRunner
from mini_infer_b200.parts import KVNeed, PlanNeeds


def runner_for(n_layers=32, pages=64 * 2100, max_requests=64, window=None, cuda_graph=True):
    needs = [SimpleNamespace(index=i, kv=KVNeed(8, 128, window), state=None) for i in range(n_layers)]
    cache = CacheManager(needs, page_size=16, num_pages=pages, max_requests=max_requests)
    model = SimpleNamespace(
        device=None, dtype=torch.bfloat16, schedule=(), graph_safe=lambda: True,
        spec=SimpleNamespace(vocab_size=128256, max_positions=131072),
        plan_needs=lambda: PlanNeeds(frozenset({16, 32, 64})))
    return StepRunner(model, cache, cuda_graph=cuda_graph), cache


def view(hp, name):
    o, n = hp.offsets[name]
    return hp.buffer[o:o + n].tolist()


def test_decode_plan_does_not_grow_with_the_context_and_is_cheap():
    sizes = {}
    for context in (64, 32768):
        runner, cache = runner_for()
        for i in range(64):
            cache.add_request(i)
            cache.plan_append([(i, context)])
        cache.take_table_updates()                      # (a real prefill step would have sent them)
        entries = [StepEntry(i, [5], [0]) for i in range(64)]
        hp = runner.host_plan(entries, graphed=True)
        sizes[context] = hp.buffer.shape[0]
        assert view(hp, "positions") == [context] * 64 and view(hp, "kv_len") == [context + 1] * 64
        # every request crossed a page edge: one new page each, as (slot, index, page) triples
        assert view(hp, "update_count0") == [64]
        triples = view(hp, "updates0")
        assert triples[0::3] == [cache.slot(i) for i in range(64)]
        assert triples[1::3] == [context // 16] * 64
        assert triples[2::3] == [cache.table(i)[-1] for i in range(64)]
    assert sizes[64] == sizes[32768]                    # bytes to the device: the same at any context
    assert sizes[64] * 4 < 8192
    best = min(_timed(runner, entries) for _ in range(20))
    assert best < 0.5e-3, f"planning a 64 x 32k decode step took {best * 1e3:.2f} ms on the host"


def _timed(runner, entries):
    t0 = time.perf_counter()
    runner.host_plan(entries, graphed=True)
    return time.perf_counter() - t0


def test_layout_of_a_mixed_step_and_of_a_captured_one():
    runner, cache = runner_for(n_layers=2, pages=64, max_requests=4)
    for r in "ab":
        cache.add_request(r)
    hp = runner.host_plan([StepEntry("a", list(range(1, 38)), [36]), StepEntry("b", [9], [0])])
    assert not hp.decode_only and hp.n_tokens == 38
    assert view(hp, "q_start") == [0, 37] and view(hp, "q_len") == [37, 1] and view(hp, "want_rows") == [36, 37]
    assert view(hp, "positions") == list(range(37)) + [0]
    assert view(hp, "state_slot") == [cache.slot("a"), cache.slot("b")]
    assert view(hp, "update_count0") == [4] and hp.update_capacity == [4]      # three pages for a, one for b
    # tiles with the most keys first: a's last tile sees 37 keys, then 32, 16, and b's one key
    assert view(hp, "tile_req16") == [0, 0, 0, 1] and view(hp, "tile_tok16") == [32, 16, 0, 0]
    # the request that brings one token is listed for the decode kernel (its row of q, its length,
    # its row of the block tables), and the tiles are listed once more without it
    assert hp.n_single == 1
    assert view(hp, "single_q_start") == [37] and view(hp, "single_kv_len") == [1]
    assert view(hp, "single_rows") == [cache.slot("b")]
    assert view(hp, "multi_req16") == [0, 0, 0] and view(hp, "multi_tok16") == [32, 16, 0] and hp.multi_counts[16] == 3
    # a captured step: fixed room for one new page per request; what is unused is marked -1
    hp = runner.host_plan([StepEntry("a", [3], [0]), StepEntry("b", [4], [0])], graphed=True)
    assert hp.decode_only and hp.update_capacity == [2] and view(hp, "update_count0") == [0]
    assert view(hp, "updates0") == [-1] * 6
    assert hp.n_single == 0 and not hp.multi_counts and view(hp, "single_q_start") == []
    # a step of prompt portions only has nobody for the decode kernel
    cache.add_request("d")
    hp = runner.host_plan([StepEntry("d", [1, 2, 3], [2])])
    assert hp.n_single == 0 and not hp.multi_counts
    cache.free_request("d")
    # pages handed out outside a step that do not fit that room travel separately
    cache.add_request("c")
    cache.plan_append([("c", 16 * 5)])
    hp = runner.host_plan([StepEntry("a", [3], [0])], graphed=True)
    assert hp.update_capacity == [1] and view(hp, "update_count0") == [0] and len(hp.overflow[0]) == 15
