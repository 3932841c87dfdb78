"""The cache manager: no page lost, held twice or freed twice, under random orders of requests;
all-or-nothing allocation; pages that a window has passed go back; state slots."""
import dataclasses
import random

import pytest

from infurnace_b200.cache import BlockPool, CacheManager, RELEASED
from infurnace_b200.config.specs import LayerCall, StateNeed
from infurnace_b200.errors import CacheError, OutOfPages
from infurnace_b200.models import config_from_dict, plan_for
import tiny


def manager(name="B", num_pages=12, max_requests=3, page_size=None):
    plan = plan_for(config_from_dict(tiny.TINY[name]["config"]))
    return CacheManager(plan, page_size or tiny.TINY[name]["page_size"], num_pages, max_requests, allocate_tensors=False)


def test_pool_hands_out_each_page_once_and_reuses_the_last_freed():
    pool = BlockPool(5)
    a = pool.allocate(3)
    assert sorted(a) == [0, 1, 2] and pool.num_free == 2
    pool.free([a[1]])
    assert pool.allocate(1) == [a[1]]            # last freed, first reused
    with pytest.raises(OutOfPages):
        pool.allocate(3)
    assert pool.num_free == 2                    # a failed allocation changes nothing
    pool.check()


def test_pool_detects_double_free_and_foreign_pages():
    pool = BlockPool(4)
    a = pool.allocate(2)
    pool.free(a)
    with pytest.raises(CacheError, match="freed twice"):
        pool.free([a[0]])
    with pytest.raises(CacheError, match="not in this pool"):
        pool.free([9])
    b = pool.allocate(1)
    with pytest.raises(CacheError, match="freed twice"):
        pool.free([b[0], b[0]])
    assert pool.is_held(b[0])                    # the bad call changed nothing
    pool.check()


def test_groups_follow_the_layers_needs():
    m = manager("B")
    assert len(m.kv_groups) == 2                 # layers 0 and 2 keep every key, layer 1 a window of 24
    full = next(g for g in m.kv_groups if g.need.window is None)
    win = next(g for g in m.kv_groups if g.need.window == 24)
    assert full.cache_ids == [0, 2] and win.cache_ids == [1]
    assert m.kv_group_of(1) != m.kv_group_of(0) == m.kv_group_of(2)
    assert len(manager("A").kv_groups) == 1


def test_allocation_is_all_or_nothing_across_groups():
    plan = plan_for(config_from_dict(tiny.TINY["B"]["config"]))
    keys = list(CacheManager(plan, 8, 4, 2, allocate_tensors=False).layout.kv)
    m = CacheManager(plan, 8, {keys[0]: 10, keys[1]: 2}, 2, allocate_tensors=False)
    m.add_request("a")
    with pytest.raises(OutOfPages):
        m.allocate("a", 17)                      # 3 pages: the second group has only 2
    assert m.free_pages() == [10, 2] and m.block_table("a", 0) == []
    m.allocate("a", 16)
    assert m.free_pages() == [8, 0]
    m.check()


def test_window_pages_are_given_back_while_the_request_runs():
    m = manager("B", num_pages=40)
    gi = next(i for i, g in enumerate(m.kv_groups) if g.need.window == 24)
    fi = 1 - gi
    m.add_request("a")
    done = 0
    for n in [30, 2, 1, 1, 50, 1]:
        m.allocate("a", n)
        assert RELEASED not in [p for p in m.block_table("a", gi)[m.kv_groups[gi].first_needed_page(done):]]
        m.slots_for("a", gi, n)                  # every new token has a live page
        m.commit("a", n)
        done += n
        first = max(0, done - 24 + 1) // 8       # the next query, at position `done`, reads from done-23
        table = m.block_table("a", gi)
        assert all(p == RELEASED for p in table[:first]) and all(p != RELEASED for p in table[first:])
        assert RELEASED not in m.block_table("a", fi)
        m.check()
    assert m.kv_groups[gi].pool.num_held <= 24 // 8 + 2
    m.free_request("a")
    assert m.free_pages() == [40, 40]


def test_release_allocation_undoes_an_uncommitted_step():
    m = manager("A", num_pages=6)
    m.add_request("a")
    m.allocate("a", 20)
    m.commit("a", 20)
    m.allocate("a", 40)
    assert m.free_pages() == [2]
    m.release_allocation("a")
    assert m.free_pages() == [4] and len(m.block_table("a", 0)) == 2
    m.check()


def test_state_slots_and_double_free_of_a_request():
    m = manager("A", max_requests=2)
    s0, s1 = m.add_request("a"), m.add_request("b")
    assert {s0, s1} == {0, 1}
    with pytest.raises(CacheError, match="no state slot"):
        m.add_request("c")
    with pytest.raises(CacheError, match="already live"):
        m.add_request("a")
    m.free_request("a")
    with pytest.raises(CacheError, match="not live"):
        m.free_request("a")
    assert m.add_request("c") == s0
    m.check()


def test_commit_without_pages_is_an_error():
    m = manager("A")
    m.add_request("a")
    with pytest.raises(CacheError, match="holds no pages"):
        m.commit("a", 3)


def test_a_layer_may_read_another_layers_cache_and_state_groups_exist():
    plan = plan_for(config_from_dict(tiny.TINY["A"]["config"]))
    shared = dataclasses.replace(plan, schedule=(LayerCall(0, cache=0), LayerCall(1, cache=0, store=False)))
    m = CacheManager(shared, 16, 4, 2, allocate_tensors=False)
    assert len(m.kv_groups) == 1 and m.kv_groups[0].cache_ids == [0]

    @dataclasses.dataclass(frozen=True)
    class StatefulLayer:
        def tensors(self):
            return {}

        def cache_need(self):
            return StateNeed((4, 3))

    mixed = dataclasses.replace(plan, layers=plan.layers + (StatefulLayer(),), schedule=plan.schedule + (LayerCall(2),))
    m = CacheManager(mixed, 16, 4, 2, allocate_tensors=False)
    assert len(m.state_groups) == 1 and m.state_group_of(2) == 0
    with pytest.raises(CacheError):
        m.kv_group_of(2)


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_the_invariants(name, seed):
    rng = random.Random(seed)
    ps = tiny.TINY[name]["page_size"]
    m = manager(name, num_pages=rng.choice([6, 9, 20]), max_requests=4)
    total = [g.pool.num_pages for g in m.kv_groups]
    live, counter = {}, 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and m.num_free_slots:
            counter += 1
            rid = f"r{counter}"
            m.add_request(rid)
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, ps, ps + 1, 3 * ps])
            before = m.free_pages()
            try:
                m.allocate(rid, n)
            except OutOfPages:
                assert m.free_pages() == before
            else:
                if rng.random() < 0.1:
                    m.release_allocation(rid)     # the step was dropped
                else:
                    slots = [m.slots_for(rid, gi, n) for gi in range(len(m.kv_groups))]
                    for gi, s in enumerate(slots):
                        assert len(set(s)) == n and all(0 <= x < total[gi] * ps for x in s)
                    m.commit(rid, n)
                    live[rid] += n
                    assert m.num_computed(rid) == live[rid]
        elif live:
            rid = rng.choice(list(live))
            m.free_request(rid)
            del live[rid]
        m.check()
        # no page is in two block tables, and free + held = total
        for gi, g in enumerate(m.kv_groups):
            held = [p for t in g.tables.values() for p in t if p != RELEASED]
            assert len(held) == len(set(held)) and len(held) + g.pool.num_free == total[gi]
    for rid in list(live):
        m.free_request(rid)
    assert m.free_pages() == total and m.num_free_slots == 4
