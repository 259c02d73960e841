"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots; all-or-nothing reservations."""

import random
from types import SimpleNamespace

import pytest

from mini_infer_b200.cache import CacheError, CacheManager, OutOfPages, PagePool
from mini_infer_b200.parts import KVNeed, StateNeed


def needs(*kv, state=None):
    return [SimpleNamespace(index=i, kv=k, state=state) for i, k in enumerate(kv)]


def full(n_layers=2):
    return needs(*[KVNeed(2, 16) for _ in range(n_layers)])


def test_pool_is_lifo_and_refuses_double_free():
    pool = PagePool(4)
    a, b = pool.allocate(), pool.allocate()
    assert (a, b) == (0, 1) and pool.num_free == 2
    pool.free(a)
    assert pool.allocate() == a          # the page given back last is handed out first
    pool.free(b)
    with pytest.raises(CacheError):
        pool.free(b)
    with pytest.raises(CacheError):
        pool.free(99)
    pool.allocate(); pool.allocate(); pool.allocate()
    with pytest.raises(OutOfPages):
        pool.allocate()


def test_block_tables_positions_and_slots():
    cm = CacheManager(full(), page_size=4, num_pages=8, max_requests=3)
    assert len(cm.groups) == 1 and cm.groups[0].layers == (0, 1)
    cm.add_request("a")
    cm.add_request("b")
    plan = cm.plan_append([("a", 6), ("b", 1)])
    assert plan.start == [0, 0] and plan.counts == [6, 1]
    ta, tb = cm.table("a"), cm.table("b")
    # the plan carries only what is new: (slot, index, page) of every page it handed out
    assert cm.take_table_updates() == [[cm.slot("a"), 0, ta[0], cm.slot("a"), 1, ta[1], cm.slot("b"), 0, tb[0]]]
    assert len(ta) == 2 and len(tb) == 1 and len(set(ta + tb)) == 3
    assert plan.token_slots[0] == [ta[0] * 4 + i for i in range(4)] + [ta[1] * 4, ta[1] * 4 + 1] + [tb[0] * 4]
    plan2 = cm.plan_append([("b", 3), ("a", 3)])          # any order, positions come from the cache
    assert plan2.start == [1, 6]
    assert plan2.token_slots[0][:3] == [tb[0] * 4 + 1, tb[0] * 4 + 2, tb[0] * 4 + 3]
    assert cm.take_table_updates() == [[cm.slot("a"), 2, cm.table("a")[2]]]   # b stayed inside its page
    assert cm.take_table_updates() == [[]]
    assert cm.length("a") == 9 and cm.length("b") == 4
    cm.check()
    cm.free_request("a")
    assert cm.num_free_pages() == 7
    cm.check()


def test_reservation_is_all_or_nothing():
    cm = CacheManager(full(), page_size=4, num_pages=3, max_requests=2)
    cm.add_request("a")
    cm.add_request("b")
    cm.plan_append([("a", 5)])
    before = (cm.length("a"), cm.length("b"), cm.num_free_pages())
    assert not cm.can_append([("a", 1), ("b", 8)])
    with pytest.raises(OutOfPages):
        cm.plan_append([("a", 1), ("b", 8)])
    assert (cm.length("a"), cm.length("b"), cm.num_free_pages()) == before
    cm.check()
    assert cm.can_append([("a", 3), ("b", 4)])
    cm.plan_append([("a", 3), ("b", 4)])
    assert cm.num_free_pages() == 0


def test_misuse_is_refused():
    cm = CacheManager(full(), page_size=4, num_pages=4, max_requests=1)
    cm.add_request("a")
    with pytest.raises(CacheError):
        cm.add_request("a")
    with pytest.raises(CacheError):
        cm.add_request("b")                         # no slot left
    with pytest.raises(CacheError):
        cm.plan_append([("zz", 1)])
    with pytest.raises(CacheError):
        cm.plan_append([("a", 0)])
    with pytest.raises(CacheError):
        cm.plan_append([("a", 1), ("a", 1)])
    cm.free_request("a")
    with pytest.raises(CacheError):
        cm.free_request("a")


def test_groups_have_pages_of_their_own_and_windows_give_pages_back():
    kinds = needs(KVNeed(2, 16), KVNeed(2, 16, window=6), KVNeed(2, 16), KVNeed(1, 32, window=6))
    cm = CacheManager(kinds, page_size=4, num_pages=[16, 5, 5], max_requests=2)
    assert [g.layers for g in cm.groups] == [(0, 2), (1,), (3,)]
    cm.add_request("a")
    held = []
    for step in range(14):
        plan = cm.plan_append([("a", 3)])
        cm.check()
        table = cm.table("a", 1)
        held.append(sum(1 for p in table if p >= 0))
        length = cm.length("a")
        # every position a later query can see (the last window-1 keys and itself) has a page
        start_of_step = length - 3
        for pos in range(max(0, start_of_step - 6 + 1), length):
            assert table[pos // 4] >= 0
        # pages wholly below the window of the step's first query are gone
        for idx in range((start_of_step - 6 + 1) // 4 if start_of_step >= 6 else 0):
            assert table[idx] == -1
    assert max(held) <= 4                       # 42 tokens went through 5 pages
    assert cm.num_free_pages(0) == 16 - 11      # the full group keeps everything
    cm.free_request("a")
    assert [cm.num_free_pages(g) for g in range(3)] == [16, 5, 5]
    cm.check()


def test_window_pages_freed_in_a_step_can_be_used_in_that_step():
    cm = CacheManager(needs(KVNeed(1, 16, window=4)), page_size=4, num_pages=3, max_requests=2)
    cm.add_request("a")
    cm.add_request("b")
    cm.plan_append([("a", 8)])
    cm.plan_append([("b", 3)])
    assert cm.num_free_pages() == 0
    # a needs a third page, and its first page has fallen out of its window: the step fits
    # only because pages are given back before new ones are taken
    assert cm.can_append([("b", 1), ("a", 1)])
    cm.plan_append([("b", 1), ("a", 1)])
    cm.check()


def test_state_slots_are_stable_and_reused():
    cm = CacheManager(needs(KVNeed(2, 16), state=StateNeed((3, 2))), page_size=4, num_pages=4, max_requests=2)
    s_a, s_b = cm.add_request("a"), cm.add_request("b")
    assert {s_a, s_b} == {0, 1}
    cm.free_request("a")
    assert cm.slot("b") == s_b                     # nobody moves when another request ends
    assert cm.add_request("c") == s_a
    cm.check()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_never_lose_or_duplicate_a_page(seed):
    rng = random.Random(seed)
    windowed = seed % 2 == 1
    kinds = needs(KVNeed(2, 16), KVNeed(2, 16, window=9 if windowed else None))
    cm = CacheManager(kinds, page_size=4, num_pages=12, max_requests=4)
    live, next_id = {}, 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and cm.num_free_slots:
            live[next_id] = 0
            cm.add_request(next_id)
            next_id += 1
        elif action < 0.4 and live:
            rid = rng.choice(list(live))
            cm.free_request(rid)
            del live[rid]
        elif live:
            chosen = rng.sample(list(live), rng.randint(1, len(live)))
            entries = [(rid, rng.choice([1, 1, 1, 2, 5, 11])) for rid in chosen]
            if cm.can_append(entries):
                plan = cm.plan_append(entries)
                for gi in range(len(cm.groups)):
                    slots = plan.token_slots[gi]
                    assert len(slots) == sum(n for _, n in entries) and len(set(slots)) == len(slots)
                for rid, n in entries:
                    live[rid] += n
            else:
                before = {rid: cm.length(rid) for rid in live}
                with pytest.raises(OutOfPages):
                    cm.plan_append(entries)
                assert before == {rid: cm.length(rid) for rid in live}
        cm.check()
        for rid, n in live.items():
            assert cm.length(rid) == n
    for rid in list(live):
        cm.free_request(rid)
    cm.check()
    assert all(cm.num_free_pages(g) == 12 for g in range(len(cm.groups)))


def test_table_updates_replay_to_the_host_tables_under_random_orders():
    """Scattering the (slot, index, page) triples in order into a table per slot, as the device
    does, gives every live request its host table (entries a window gave back aside)."""
    rng = random.Random(3)
    kinds = needs(KVNeed(2, 16), KVNeed(2, 16, window=9))
    cm = CacheManager(kinds, page_size=4, num_pages=[24, 8], max_requests=4, max_request_tokens=400)
    assert cm.table_width == [24, 100]
    device = [dict() for _ in cm.groups]            # (slot, index) -> page
    live, next_id = [], 0
    for _ in range(300):
        action = rng.random()
        if action < 0.3 and cm.num_free_slots:
            cm.add_request(next_id)
            live.append(next_id)
            next_id += 1
        elif action < 0.45 and live:
            cm.free_request(live.pop(rng.randrange(len(live))))
        elif live:
            entries = [(rid, rng.choice([1, 1, 2, 7])) for rid in rng.sample(live, rng.randint(1, len(live)))]
            if cm.can_append(entries):
                cm.plan_append(entries)
        for gi, flat in enumerate(cm.take_table_updates()):
            assert len(flat) % 3 == 0
            for i in range(0, len(flat), 3):
                device[gi][(flat[i], flat[i + 1])] = flat[i + 2]
        for rid in live:
            for gi in range(len(cm.groups)):
                for idx, page in enumerate(cm.table(rid, gi)):
                    if page >= 0:
                        assert device[gi][(cm.slot(rid), idx)] == page


def test_a_request_longer_than_its_block_table_is_refused():
    cm = CacheManager(full(), page_size=4, num_pages=64, max_requests=2, max_request_tokens=20)
    assert cm.table_width == [5]
    cm.add_request("a")
    cm.plan_append([("a", 19)])
    with pytest.raises(CacheError, match="block table"):
        cm.plan_append([("a", 2)])
    assert cm.length("a") == 19
    cm.plan_append([("a", 1)])
    cm.check()
