"""The scheduler's decisions (no GPU): admission, portions, budget, preemption, refusal."""
import pytest

from safetyraise_lmengine_b200.cache.manager import PAGED_ALL, CacheGroupSpec, CacheManager
from safetyraise_lmengine_b200.engine.scheduler import Scheduler
from safetyraise_lmengine_b200.errors import ConfigError, ResourceExhausted

KV = CacheGroupSpec("kv", PAGED_ALL, (0,), kv_heads=1, head_dim=16)


def make(num_pages=64, page=4, max_active=4, queue=8, chunk=8, budget=16, context=128):
    cache = CacheManager([KV], page_size=page, num_pages=num_pages, max_requests=max_active)
    return cache, Scheduler(cache, max_active, queue, chunk, budget, context)


def run_step(s, plan, sample=True):
    """Pretend the step ran: advance everything, then add one token where logits were wanted."""
    for p in plan:
        s.advance(p.request_id, p.count)
    done = []
    for p in plan:
        if p.want_logits:
            done.append(p.request_id)
            if sample:
                s.append_token(p.request_id)
    return done


def test_prompt_is_cut_into_portions_under_the_budget():
    cache, s = make(chunk=8, budget=12)
    s.submit(1, 20, 4)
    s.submit(2, 5, 4)
    plan, _ = s.plan()
    assert [(p.request_id, p.start, p.count, p.want_logits) for p in plan] == [(1, 0, 8, False), (2, 0, 4, False)]
    run_step(s, plan)
    plan, _ = s.plan()
    assert [(p.request_id, p.start, p.count, p.want_logits) for p in plan] == [(1, 8, 8, False), (2, 4, 1, True)]
    run_step(s, plan)
    plan, _ = s.plan()     # request 2 decodes (first in the batch), request 1 ends its prompt
    assert [(p.request_id, p.start, p.count, p.want_logits) for p in plan] == [(2, 5, 1, True), (1, 16, 4, True)]
    assert s.counters()["batched_tokens"] == 12 + 9 + 5


def test_submit_refusals():
    cache, s = make(num_pages=4, page=4, queue=2, context=32)
    with pytest.raises(ConfigError):
        s.submit(1, 0, 4)
    with pytest.raises(ConfigError):
        s.submit(1, 30, 4)                       # longer than the context
    with pytest.raises(ResourceExhausted):
        s.submit(1, 14, 4)                       # 18 tokens need 5 pages, the pool has 4
    s.submit(1, 4, 4)
    s.submit(2, 4, 4)
    with pytest.raises(ResourceExhausted):
        s.submit(3, 4, 4)                        # queue of 2 is full
    with pytest.raises(ConfigError):
        s.submit(2, 4, 4)                        # duplicate id
    c = s.counters()
    assert c["rejected"] == 5 and c["queued"] == 2


def test_max_active_and_finish_frees():
    cache, s = make(max_active=2)
    for i in (1, 2, 3):
        s.submit(i, 4, 2)
    plan, _ = s.plan()
    assert {p.request_id for p in plan} == {1, 2} and s.counters()["queued"] == 1
    run_step(s, plan)
    s.finish(1)
    assert cache.audit() == 0
    plan, _ = s.plan()
    assert {p.request_id for p in plan} == {2, 3}
    for i in (2, 3):
        s.finish(i)
    assert not s.has_work() and cache.free_pages("kv") == 64 and cache.audit() == 0


def test_preempts_the_youngest_when_a_decode_finds_no_page():
    # 4 pages of 4 tokens; two requests of prompt 7 fill all pages; decoding past 8 needs a third page each
    cache, s = make(num_pages=4, page=4, chunk=8, budget=16)
    s.submit(1, 7, 6)
    s.submit(2, 7, 6)
    plan, pre = s.plan()
    assert [(p.request_id, p.count) for p in plan] == [(1, 7), (2, 7)] and pre == []
    run_step(s, plan)                            # both now hold 8 tokens in all, 7 in the cache
    plan, pre = s.plan()
    assert [p.count for p in plan] == [1, 1] and pre == []
    run_step(s, plan)                            # 9 tokens in all each; the next token needs page 3 of each
    plan, pre = s.plan()
    assert pre == [2]                            # the youngest gives way
    assert [(p.request_id, p.start, p.count) for p in plan] == [(1, 8, 1)]
    assert cache.audit() == 0 and s.counters()["preempted"] == 1
    run_step(s, plan)
    # request 2 waits at the head of the queue: one free page does not hold its first portion
    for _ in range(3):
        plan, pre = s.plan()
        assert [p.request_id for p in plan] == [1] and pre == []
        run_step(s, plan)
    s.finish(1)
    plan, pre = s.plan()     # it comes back with its prompt and its 2 generated tokens, from 0
    assert [(p.request_id, p.start, p.count, p.want_logits) for p in plan] == [(2, 0, 8, False)]
    run_step(s, plan)
    plan, _ = s.plan()
    assert (plan[0].start, plan[0].count, plan[0].want_logits) == (8, 1, True)           # 9 tokens in all
    s.finish(2)
    assert cache.free_pages("kv") == 4 and cache.audit() == 0


def test_blocked_prompts_make_the_youngest_give_way():
    # two prompts of 12 tokens share 4 pages of 4: after two portions each, neither finds a page
    cache, s = make(num_pages=4, page=4, chunk=4, budget=8, max_active=2)
    s.submit(1, 12, 2)
    s.submit(2, 12, 2)
    for _ in range(2):
        plan, pre = s.plan()
        assert [(p.request_id, p.count) for p in plan] == [(1, 4), (2, 4)] and pre == []
        run_step(s, plan)
    plan, pre = s.plan()
    assert pre == [2]                            # the oldest keeps its pages and goes on
    assert [(p.request_id, p.start, p.count, p.want_logits) for p in plan] == [(1, 8, 4, True)]
    assert cache.audit() == 0


def test_every_request_ends_under_pressure():
    cache, s = make(num_pages=6, page=4, chunk=5, budget=9, max_active=3, queue=16)
    want = {i: (3 + 2 * i, 5) for i in range(1, 9)}       # (prompt, max_new)
    for i, (p, n) in want.items():
        s.submit(i, p, n)
    generated = {i: 0 for i in want}
    finished = set()
    for _ in range(2000):
        if not s.has_work():
            break
        plan, _ = s.plan()
        assert plan, "the scheduler must always find something to run"
        assert sum(p.count for p in plan) <= 9
        for p in plan:
            s.advance(p.request_id, p.count)
        for p in plan:
            if p.want_logits:
                generated[p.request_id] = s.append_token(p.request_id)
                if generated[p.request_id] >= want[p.request_id][1]:
                    s.finish(p.request_id)
                    finished.add(p.request_id)
        assert cache.audit() == 0
    assert finished == set(want) and cache.free_pages("kv") == 6
    assert s.counters()["preempted"] > 0


def test_retract_token_undoes_an_unfed_token():
    """A token that was counted before its value was known (the next step is laid out while the device
    still samples) and turns out to be a stop token is taken back: lengths and counters as before."""
    cache, sched = make(num_pages=8, page=4)
    sched.submit(1, 5, 4)
    plan, _ = sched.plan()
    assert [(p.start, p.count, p.want_logits) for p in plan] == [(0, 5, True)]
    sched.advance(1, 5)
    assert sched.append_token(1) == 1
    before = sched.counters()["generated_tokens"]
    assert sched.retract_token(1) == 0
    assert sched.counters()["generated_tokens"] == before - 1
    assert sched.retract_token(1) < 0                     # nothing left to take back
    assert sched.append_token(1) == 1                     # and it can be counted again
    plan, _ = sched.plan()
    assert [(p.start, p.count) for p in plan] == [(5, 1)]
    sched.finish(1)
    assert cache.audit() == 0
