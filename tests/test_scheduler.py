"""The scheduler's decisions on the CPU, driven by a fake step that only keeps the cache's
books: token budget, decode first, portions, finish reasons, and what happens when pages run out."""
import pytest
import torch

from hfee_b200.cache import CacheManager, PagedKV
from hfee_b200.engine.scheduler import FinishReason, Request, Scheduler
from hfee_b200.sampling import SamplingOptions


def make(num_pages=16, page=4, reqs=4, ctx=64, budget=32, chunk=None, eos=()):
    cache = CacheManager({0: PagedKV(1, 8)}, page, num_pages, reqs, ctx, torch.float32, "cpu")
    return cache, Scheduler(cache, budget, chunk, eos)


def req(i, n_prompt, num_predict=-1):
    return Request(id=i, prompt=list(range(1, n_prompt + 1)), options=SamplingOptions.greedy(num_predict))


def run_plan(cache, sched, plan, next_token=lambda r: 100 + len(r.output)):
    """What the runner does to the cache for a plan, plus scripted sampling."""
    for e in plan:
        new = cache.length[e.request.slot] + len(e.tokens)
        cache.reserve(e.request.slot, new)
        cache.commit(e.request.slot, new)
    sched.update(plan, [next_token(e.request) for e in plan if e.wants_logits])
    cache.check_invariants()


def test_budget_portions_and_decode_first():
    cache, s = make(budget=16, num_pages=64, ctx=200)
    a, b = req("a", 40), req("b", 5)
    s.add(a); s.add(b)
    plan = s.plan()                                   # prompts in admission order under the budget
    assert [(e.request.id, len(e.tokens), e.wants_logits) for e in plan] == [("a", 16, False)]
    run_plan(cache, s, plan)
    plan = s.plan()
    assert [(e.request.id, len(e.tokens)) for e in plan] == [("a", 16)]
    run_plan(cache, s, plan)
    plan = s.plan()                                   # a's last 8 tokens, then b's whole prompt
    assert [(e.request.id, len(e.tokens), e.wants_logits) for e in plan] == [("a", 8, True), ("b", 5, True)]
    run_plan(cache, s, plan)
    assert a.decoding and b.decoding and a.output == [100] and a.feed == [100]
    c = req("c", 30)
    s.add(c)
    plan = s.plan()                                   # decoding requests first, one token each, then c's portion
    assert [(e.request.id, len(e.tokens)) for e in plan] == [("a", 1), ("b", 1), ("c", 14)]
    assert plan[0].tokens == [100]


def test_prefill_chunk_limits_a_portion():
    cache, s = make(budget=32, chunk=6, num_pages=64)
    s.add(req("a", 20))
    assert [len(e.tokens) for e in s.plan()] == [6]


def test_finish_reasons_and_pages_freed():
    cache, s = make(eos=(7,))
    a, b = req("a", 3, num_predict=2), req("b", 3)
    s.add(a); s.add(b)
    run_plan(cache, s, s.plan())
    run_plan(cache, s, s.plan(), next_token=lambda r: 7 if r is b else 50)
    assert a.finished == FinishReason.LENGTH and a.output == [100, 50] and a.stats.eval_tokens == 2
    assert b.finished == FinishReason.STOP and b.output == [100]       # the end token is not emitted
    assert sorted(r.id for r in s.pop_finished()) == ["a", "b"] and s.idle
    assert cache.free_pages() == 16 and cache.free_slots() == 4


def test_context_limit_ends_with_length():
    cache, s = make(ctx=8, num_pages=16)
    with pytest.raises(ValueError, match="context window"):
        s.add(req("big", 8))
    a = req("a", 6)
    s.add(a)
    for _ in range(5):
        plan = s.plan()
        if not plan:
            break
        run_plan(cache, s, plan)
    assert a.finished == FinishReason.LENGTH and cache.length == [0] * 4
    assert len(a.prompt) + len(a.output) <= 8 + 1


def test_waits_for_a_slot_fifo():
    cache, s = make(reqs=2)
    rs = [req(i, 2, num_predict=1) for i in range(4)]
    for r in rs:
        s.add(r)
    plan = s.plan()
    assert [e.request.id for e in plan] == [0, 1] and len(s.waiting) == 2
    run_plan(cache, s, plan)                                            # both finish (num_predict 1)
    assert [e.request.id for e in s.plan()] == [2, 3]


def test_out_of_pages_preempts_the_last_admitted_and_recomputes():
    cache, s = make(num_pages=4, page=4, budget=64, ctx=64)            # 16 tokens of cache in all
    a, b = req("a", 7), req("b", 7)
    s.add(a); s.add(b)
    run_plan(cache, s, s.plan())                                        # 2 pages each: the pool is full
    assert cache.free_pages() == 0
    run_plan(cache, s, s.plan())                                        # 8th token of each fits its page
    assert len(a.output) == len(b.output) == 2 and s.preemptions == 0
    plan = s.plan()                                                     # both need a third page; none is free
    assert s.preemptions == 1 and b.slot is None and s.waiting[0] is b
    assert b.feed == b.prompt + b.output and not b.decoding and b.stats.preemptions == 1
    assert [e.request.id for e in plan] == ["a"]
    run_plan(cache, s, plan)
    # b stays out while it does not fit; a keeps decoding until it ends
    a.options = a.options.with_(num_predict=len(a.output) + 1)
    run_plan(cache, s, s.plan())
    assert a.finished == FinishReason.LENGTH
    plan = s.plan()                                                     # b comes back and recomputes everything
    assert [(e.request.id, len(e.tokens), e.wants_logits) for e in plan] == [("b", 9, True)]
    run_plan(cache, s, plan)
    assert b.decoding and len(b.output) == 3 and b.draws == 3           # sampling counters went on


def test_a_request_that_cannot_fit_alone_ends_with_length():
    cache, s = make(num_pages=2, page=4, budget=64, ctx=64)
    a = req("a", 6)
    s.add(a)
    for _ in range(10):
        plan = s.plan()
        if not plan:
            break
        run_plan(cache, s, plan)
    assert a.finished == FinishReason.LENGTH and len(a.prompt) + len(a.output) == 9   # 8 cached + the last sampled
    assert cache.free_pages() == 2 and s.idle


def test_admission_waits_for_the_first_portions_pages():
    cache, s = make(num_pages=5, page=4, budget=64, ctx=64)
    a, b = req("a", 11), req("b", 12)
    s.add(a); s.add(b)
    plan = s.plan()                                    # a takes 3 pages; b's 3 pages do not fit beside it
    assert [(e.request.id, len(e.tokens)) for e in plan] == [("a", 11)] and list(s.waiting) == [b]
    run_plan(cache, s, plan)
    assert [e.request.id for e in s.plan()] == ["a"] and list(s.waiting) == [b]
    c = req("c", 8)
    s.add(c)
    s.waiting.rotate(1)                                # a shorter one at the head of the queue fits
    plan = s.plan()
    assert [(e.request.id, len(e.tokens)) for e in plan] == [("a", 1), ("c", 8)] and list(s.waiting) == [b]


def test_a_lone_prompt_larger_than_the_cache_is_cut_to_it_then_ends():
    cache, s = make(num_pages=5, page=4, budget=64, ctx=64)
    a = req("a", 30)
    s.add(a)
    plan = s.plan()                                    # nothing else runs: admitted, portion cut to 20 tokens
    assert [(e.request.id, len(e.tokens), e.wants_logits) for e in plan] == [("a", 20, False)]
    run_plan(cache, s, plan)
    assert s.plan() == [] and a.finished == FinishReason.LENGTH and cache.free_pages() == 5


def test_abort_frees_and_reports():
    cache, s = make()
    a, b = req("a", 5), req("b", 5)
    s.add(a); s.add(b)
    run_plan(cache, s, s.plan())
    s.abort(a)
    assert a.finished == FinishReason.ABORT and cache.free_slots() == 3
    c = req("c", 3)
    s.add(c)
    s.abort(c)
    assert c.finished == FinishReason.ABORT and [r.id for r in s.pop_finished()] == ["a", "c"]


def test_provisional_updates_resolve_one_step_late():
    from hfee_b200.engine.scheduler import DEVICE_TOKEN
    cache, s = make(eos=(7,))
    a, b, c = req("a", 3, num_predict=3), req("b", 3), req("c", 3)
    for r in (a, b, c):
        s.add(r)

    def launch():
        plan = s.plan()
        for e in plan:
            new = cache.length[e.request.slot] + len(e.tokens)
            cache.reserve(e.request.slot, new)
            cache.commit(e.request.slot, new)
        return s.update_provisional(plan)

    p0 = launch()                                  # prompts; tokens unknown yet
    assert [r.id for r, _ in p0] == ["a", "b", "c"] and a.output == [DEVICE_TOKEN] and a.feed == [DEVICE_TOKEN]
    p1 = launch()                                  # launched before p0 is known: inputs are placeholders
    assert all(e == [DEVICE_TOKEN] for e in (a.feed, b.feed, c.feed))
    s.resolve(p0, [50, 7, 51])                     # b's first token was an end token
    assert a.output == [50, DEVICE_TOKEN] and b.output == [] and b.finished == FinishReason.STOP
    assert b.stats.eval_tokens == 0 and c.output == [51, DEVICE_TOKEN]
    p2 = launch()                                  # b is gone; a reaches num_predict = 3 and ends provisionally
    assert [r.id for r, _ in p2] == ["a", "c"] and a.finished == FinishReason.LENGTH
    s.resolve(p1, [60, 61, 62])                    # b's row is ignored: its output was cut
    assert a.output == [50, 60, DEVICE_TOKEN] and b.output == [] and c.output == [51, 62, DEVICE_TOKEN]
    s.resolve(p2, [7, 63])                         # a's third token turns out to be an end token
    assert a.output == [50, 60] and a.finished == FinishReason.STOP and a.stats.eval_tokens == 2
    assert c.output == [51, 62, 63]
    cache.check_invariants()
