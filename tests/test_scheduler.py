"""The scheduler's decisions, on numbers only: a cache manager without tensors and a step
function that only does the accounting."""
import pytest

from infurnace_b200.cache import CacheManager
from infurnace_b200.engine.request import Request, RequestState, SamplingParams
from infurnace_b200.engine.scheduler import Scheduler
from infurnace_b200.errors import SchedulerError
from infurnace_b200.models import config_from_dict, plan_for
import tiny


def make(num_pages=64, max_seqs=4, budget=32, max_len=128, name="A", portion=None):
    plan = plan_for(config_from_dict(tiny.TINY[name]["config"]))
    cache = CacheManager(plan, tiny.TINY[name]["page_size"], num_pages, max_seqs, allocate_tensors=False)
    return Scheduler(cache, max_seqs, budget, max_len, portion), cache


def req(rid, n, max_tokens=8, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, **kw))


def run_step(s, cache, token=7):
    """Plan a step, do the cache accounting the step function does, and commit it."""
    plan = s.schedule()
    for e in plan.entries:
        cache.allocate(e.request_id, len(e.tokens))
    for e in plan.entries:
        cache.commit(e.request_id, len(e.tokens))
        s.advance(e)
        if e.sample:
            r = s.get_request(e.request_id)
            r.append_output_token(token)
            s.on_token(e.request_id)
            reason = r.check_finished(token)
            if reason:
                s.finish(e.request_id, reason)
    cache.check()
    return plan


def test_admission_rules():
    s, _ = make(max_len=20)
    s.add_request(req("ok", 10, 10))
    s.add_request(req("long", 21, 1))
    s.add_request(req("sum", 15, 6))
    s.add_request(Request("limit", [1] * 8, SamplingParams(max_tokens=4), context_limit=10))
    s.add_request(req("empty", 0))
    s.add_request(req("topk", 3, top_k=5))
    s.add_request(req("topp", 3, top_p=0.9))
    assert s.get_request("ok").state is RequestState.WAITING
    assert "exceeds context limit 20" in s.get_request("long").error
    assert "max_tokens 6 exceeds" in s.get_request("sum").error
    assert "context limit 10" in s.get_request("limit").error
    for rid in ("long", "sum", "limit", "empty", "topk", "topp"):
        assert s.get_request(rid).state is RequestState.REJECTED
    with pytest.raises(SchedulerError, match="duplicate"):
        s.add_request(req("ok", 3))
    with pytest.raises(SchedulerError):
        Scheduler(_, 0, 1, 1)


def test_prompts_are_cut_into_portions_under_the_budget():
    s, cache = make(budget=32)
    s.add_request(req("a", 70))
    plans = drain(s, cache, until=lambda: s.get_request("a").state is RequestState.DECODING)
    sizes = [[(e.start, len(e.tokens), e.sample) for e in plan.entries] for plan in plans]
    assert sizes == [[(0, 32, False)], [(32, 32, False)], [(64, 6, True)]]
    assert s.get_request("a").state is RequestState.DECODING


def test_decode_goes_first_and_prefill_takes_the_rest():
    s, cache = make(budget=16)
    s.add_request(req("a", 4))
    run_step(s, cache)                                   # a: whole prompt, first token
    s.add_request(req("b", 40))
    plan = run_step(s, cache)
    assert [(e.request_id, len(e.tokens)) for e in plan.entries] == [("a", 1), ("b", 15)]
    plan = run_step(s, cache)
    assert [(e.request_id, e.start, len(e.tokens)) for e in plan.entries] == [("a", 5, 1), ("b", 15, 15)]
    assert plan.num_tokens == 16


def test_fifo_admission_and_the_limit_on_live_requests():
    s, cache = make(max_seqs=2, budget=64)
    for i in range(4):
        s.add_request(req(f"r{i}", 5, max_tokens=2))
    plan = run_step(s, cache)
    assert [e.request_id for e in plan.entries] == ["r0", "r1"] and s.num_waiting == 2
    plan = run_step(s, cache)                            # both finish with their second token
    assert s.get_request("r0").state is RequestState.FINISHED
    plan = run_step(s, cache)
    assert [e.request_id for e in plan.entries] == ["r2", "r3"]


def test_max_prefill_portion():
    s, cache = make(budget=64, portion=10)
    s.add_request(req("a", 25))
    s.add_request(req("b", 25))
    plan = run_step(s, cache)
    assert [(e.request_id, len(e.tokens)) for e in plan.entries] == [("a", 10), ("b", 10)]


def test_decode_positions_and_tokens():
    s, cache = make()
    s.add_request(req("a", 3))
    run_step(s, cache, token=50)
    plan = s.schedule()
    e = plan.entries[0]
    # the last token is fed back at the position equal to the sequence length so far minus one
    # (the reference's decode plan: src/infurnace/scheduler/scheduler.py:160-172)
    assert e.tokens == (50,) and e.start == 3 and e.sample


def drain(s, cache, until=None, limit=300):
    """Run steps until ``until()`` holds (default: the scheduler is idle); never forever."""
    plans = []
    for _ in range(limit):
        if (until or (lambda: s.is_idle))():
            return plans
        plans.append(run_step(s, cache))
    raise AssertionError("the scheduler did not get there in %d steps" % limit)


def test_when_pages_run_out_the_last_admitted_request_is_preempted():
    # pages of 16 tokens, 3 pages: "old" (20 + 8 tokens) holds 2 for all its life, "new" (14 + 30) needs 3
    s, cache = make(num_pages=3, budget=64, max_len=100)
    s.add_request(req("old", 20, max_tokens=8))
    s.add_request(req("new", 14, max_tokens=30))
    plan = run_step(s, cache)
    assert [e.request_id for e in plan.entries] == ["old", "new"]       # 2 + 1 pages, none free
    for _ in range(2):
        run_step(s, cache)                                              # new reaches 16 tokens: its page is full
    plan = run_step(s, cache)                                           # new needs a 2nd page: none left
    assert plan.preempted == ["new"] and [e.request_id for e in plan.entries] == ["old"]
    new = s.get_request("new")
    assert new.state is RequestState.WAITING and new.num_computed_tokens == 0 and new.num_preemptions == 1
    assert len(new.output_token_ids) == 3                               # it keeps what it generated
    assert cache.free_pages() == [1]
    # it comes back from position 0 and recomputes prompt and generated tokens
    plan = run_step(s, cache)
    e = next(e for e in plan.entries if e.request_id == "new")
    assert e.start == 0 and e.tokens == tuple(new.all_token_ids[:16]) and not e.sample
    plans = drain(s, cache)
    assert s.get_request("old").state is RequestState.FINISHED
    assert new.state is RequestState.FINISHED and len(new.output_token_ids) == 30
    assert cache.free_pages() == [3]


def test_the_victim_is_the_last_admitted_even_if_it_is_the_one_asking():
    s, cache = make(num_pages=4, budget=64, max_len=100)
    s.add_request(req("a", 16, max_tokens=40))       # 1 page, needs a 2nd at once
    s.add_request(req("b", 30, max_tokens=40))       # 2 pages
    run_step(s, cache)                               # a: 1 page, b: 2 pages -> 1 free
    plan = run_step(s, cache)                        # a takes the last page (decode goes in admission order)
    assert not plan.preempted
    for _ in range(2):
        plan = run_step(s, cache)                    # b reaches 32 tokens and needs a 3rd page
    assert plan.preempted == ["b"]
    assert [e.request_id for e in plan.entries] == ["a"]


def test_a_lone_request_that_cannot_advance_fails():
    s, cache = make(num_pages=2, budget=64, max_len=100)
    s.add_request(req("a", 30, max_tokens=20))
    drain(s, cache, until=lambda: s.get_request("a").is_terminal())
    r = s.get_request("a")
    assert r.state is RequestState.FAILED and r.error == "out of KV pages" and len(r.output_token_ids) == 3
    assert cache.free_pages() == [2] and s.is_idle


def test_a_prompt_larger_than_the_pool_fails_instead_of_waiting_forever():
    s, cache = make(num_pages=2, budget=16, max_len=100)
    s.add_request(req("big", 50))
    states = []
    for _ in range(6):
        run_step(s, cache)
        states.append(s.get_request("big").state)
    assert states[-1] is RequestState.FAILED and s.is_idle and cache.free_pages() == [2]


def test_waiting_requests_wait_for_pages():
    s, cache = make(num_pages=2, budget=64, max_len=100)
    s.add_request(req("a", 20, max_tokens=5))
    s.add_request(req("b", 20, max_tokens=5))
    plan = run_step(s, cache)
    assert [e.request_id for e in plan.entries] == ["a"] and s.num_waiting == 1
    drain(s, cache, until=lambda: s.get_request("a").state is RequestState.FINISHED)
    assert run_step(s, cache).entries[0].request_id == "b"


def test_cancel_frees_at_once_and_is_idempotent():
    s, cache = make()
    s.add_request(req("a", 20))
    s.add_request(req("b", 5))
    run_step(s, cache)
    s.cancel("a")
    s.cancel("a")
    assert s.get_request("a").state is RequestState.CANCELLED and not cache.has_request("a")
    s.cancel("b")
    assert s.is_idle and cache.free_pages() == [64]
    s.add_request(req("c", 5))
    s.cancel("c")                                        # cancelled while waiting
    assert s.schedule().entries == []


def test_stop_rules_in_the_references_order():
    r = Request("x", [1, 2], SamplingParams(max_tokens=3, stop_token_ids=[9], min_tokens=2), eos_token_ids=[5])
    r.append_output_token(5)
    assert r.check_finished(5) is None                   # the min_tokens floor suppresses eos
    r.append_output_token(5)
    assert r.check_finished(5) == "eos"
    assert r.check_finished(9) == "stop_token_ids"
    r.append_output_token(1)
    assert r.check_finished(1) == "max_tokens"
    z = Request("z", [1], SamplingParams(max_tokens=0))
    z.append_output_token(4)
    assert z.check_finished(4) == "max_tokens"           # the first token always counts


def test_transitions():
    r = Request("x", [1])
    with pytest.raises(ValueError):
        r.transition(RequestState.DECODING)
    r.transition(RequestState.PREFILLING)
    r.transition(RequestState.WAITING)                   # preemption
    r.transition(RequestState.PREFILLING)
    r.transition(RequestState.DECODING)
    r.transition(RequestState.FINISHED)
    assert r.metrics.completion_time is not None
    with pytest.raises(ValueError):
        r.transition(RequestState.CANCELLED)
