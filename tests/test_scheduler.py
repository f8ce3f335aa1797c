"""The scheduler's decisions, with a cache manager and no model (the step is faked)."""

import pytest

from qwen3_from_scratch_b200.cache import CacheManager, layout_of
from qwen3_from_scratch_b200.engine.request import Request, RequestStatus, SamplingParams
from qwen3_from_scratch_b200.engine.scheduler import Scheduler, SchedulerConfig
from qwen3_from_scratch_b200.parts.base import KVCacheSpec


def make(num_pages=64, page_size=4, max_num_seqs=4, max_num_tokens=32, chunk=16, specs=None):
    specs = specs or [KVCacheSpec(2, 16, None)]
    cache = CacheManager(layout_of(dict(enumerate(specs))), page_size, num_pages, max_num_seqs)
    sched = Scheduler(SchedulerConfig(max_num_seqs, max_num_tokens, chunk), cache)
    return sched, cache


def req(n_prompt, max_new=4, **kw):
    return Request(list(range(1, n_prompt + 1)), SamplingParams(max_new_tokens=max_new, **kw))


def run_step(sched, token=7):
    plan = sched.schedule()
    finished = sched.post_process(plan, [token if s.wants_logits else None for s in plan])
    sched.cache.check()
    return plan, finished


def summary(plan):
    return [(s.request.request_id, s.num_tokens, s.wants_logits) for s in plan]


def test_request_that_can_never_fit_is_refused():
    sched, _ = make(num_pages=4, page_size=4)
    assert not sched.add_request(req(10, max_new=7))  # 17 > 16 tokens of cache
    assert sched.add_request(req(10, max_new=6))
    sched.config.max_positions = 12
    assert not sched.add_request(req(10, max_new=6))


def test_prompt_is_cut_into_portions_under_the_token_budget():
    sched, cache = make(max_num_tokens=32, chunk=16)
    a = req(40)
    sched.add_request(a)
    plan, _ = run_step(sched)
    assert summary(plan) == [(a.request_id, 16, False)] and a.num_computed == 16
    plan, _ = run_step(sched)
    assert summary(plan) == [(a.request_id, 16, False)]
    plan, _ = run_step(sched)
    assert summary(plan) == [(a.request_id, 8, True)] and a.output == [7]
    plan, _ = run_step(sched)
    assert summary(plan) == [(a.request_id, 1, True)] and a.is_decoding is False or True
    assert cache.length(a) == 41


def test_decodes_first_then_running_prompts_then_new_requests():
    sched, _ = make(max_num_tokens=20, chunk=16, max_num_seqs=4)
    a, b, c = req(3), req(30), req(5)
    sched.add_request(a)
    run_step(sched)            # a finishes its prompt and has one token
    sched.add_request(b)
    run_step(sched)            # a decodes, b gets a portion
    sched.add_request(c)
    plan = sched.schedule()
    # a: one token; b: the rest of the budget (up to its chunk); c: whatever is left
    assert summary(plan)[0] == (a.request_id, 1, True)
    assert summary(plan)[1] == (b.request_id, 14, True)
    assert summary(plan)[2] == (c.request_id, 5, True)
    assert sum(s.num_tokens for s in plan) <= 20


def test_sequence_budget_limits_a_step():
    sched, _ = make(max_num_seqs=2, max_num_tokens=100)
    reqs = [req(4) for _ in range(3)]
    for r in reqs:
        sched.add_request(r)
    plan, _ = run_step(sched)
    assert [s.request for s in plan] == reqs[:2]
    assert reqs[2].status == RequestStatus.WAITING


def test_finish_by_length_and_by_eos_frees_everything():
    sched, cache = make()
    sched.is_finished = lambda r: ("eos" if r.output[-1] == 99 else
                                   "length" if len(r.output) >= r.params.max_new_tokens else None)
    a, b = req(5, max_new=2), req(6, max_new=50)
    sched.add_request(a)
    sched.add_request(b)
    run_step(sched)
    _, finished = run_step(sched)
    assert finished == [a] and a.finish_reason == "length" and a.status == RequestStatus.FINISHED
    _, finished = run_step(sched, token=99)
    assert finished == [b] and b.finish_reason == "eos"
    assert not sched.has_work() and cache.free_pages() == 64 and cache.free_slots() == 4


def test_decode_out_of_pages_preempts_the_newest_decoding_request():
    sched, cache = make(num_pages=4, page_size=4, max_num_tokens=64, chunk=64)
    a, b = req(7, max_new=8), req(7, max_new=8)
    sched.add_request(a)
    sched.add_request(b)
    run_step(sched)  # both prompts: 2 pages each, the pool is full; both now hold 7 tokens
    plan, _ = run_step(sched)  # position 7 fits in the second page of each
    assert len(plan) == 2
    plan = sched.schedule()  # position 8 needs a third page: none free -> b (newest) is preempted
    assert [s.request for s in plan] == [a]
    assert b.status == RequestStatus.WAITING and b.num_computed == 0 and b.preemptions == 1
    assert b.output == [7, 7], "a preempted request keeps what it generated"
    assert sched.waiting[0] is b, "and waits at the front"
    sched.post_process(plan, [7])
    cache.check()
    # b comes back once a has finished, recomputing prompt + generated
    for _ in range(40):
        if not sched.has_work():
            break
        run_step(sched)
    assert a.status == b.status == RequestStatus.FINISHED
    assert len(a.output) == len(b.output) == 8
    assert cache.free_pages() == 4


def test_last_decoding_request_preempts_itself_when_a_prompt_holds_the_pages():
    sched, cache = make(num_pages=4, page_size=4, max_num_tokens=64, chunk=8)
    a = req(3, max_new=12)
    sched.add_request(a)
    run_step(sched)
    b = req(12, max_new=1)
    sched.add_request(b)
    run_step(sched)  # a decodes (4 tokens = 1 page), b's first 8 tokens take 2 pages
    run_step(sched)  # a needs page 2 (1 left), b's last 4 tokens need 1 more: a is served first
    assert b.status == RequestStatus.RUNNING
    for _ in range(60):
        if not sched.has_work():
            break
        run_step(sched)
    assert a.status == b.status == RequestStatus.FINISHED
    assert len(a.output) == 12 and len(b.output) == 1


def test_portion_without_pages_waits_and_blocks_admission():
    sched, cache = make(num_pages=6, page_size=4, max_num_tokens=64, chunk=8)
    a, b, c = req(16, max_new=1), req(16, max_new=1), req(2, max_new=1)
    sched.add_request(a)
    sched.add_request(b)
    run_step(sched)  # a: 8 tokens (2 pages), b: 8 tokens (2 pages); 2 pages left
    sched.add_request(c)
    plan = sched.schedule()
    # a takes the last 2 pages, b's portion has to wait, and c is not admitted past it
    assert [s.request for s in plan] == [a]
    assert c.status == RequestStatus.WAITING
    sched.post_process(plan, [7])
    for _ in range(20):
        if not sched.has_work():
            break
        run_step(sched)
    assert all(r.status == RequestStatus.FINISHED for r in (a, b, c))


def test_two_prompts_that_block_each_other_are_untangled():
    sched, cache = make(num_pages=6, page_size=4, max_num_tokens=16, chunk=8)
    a, b = req(20, max_new=1), req(20, max_new=1)  # each needs 5 pages for its prompt, 6 in all
    sched.add_request(a)
    sched.add_request(b)
    steps = 0
    while sched.has_work():
        plan, _ = run_step(sched)
        assert plan, "the scheduler must always find something to run"
        steps += 1
        assert steps < 50
    assert sched.num_preemptions >= 1
    assert a.status == b.status == RequestStatus.FINISHED


def test_window_layers_let_a_long_request_run_in_a_small_pool():
    """With a window in every layer, pages come back while the request grows."""
    sched, cache = make(num_pages=5, page_size=4, max_num_tokens=8, chunk=4,
                        specs=[KVCacheSpec(2, 16, 6)])
    a = req(10, max_new=10)  # 20 tokens = 5 pages: admitted, but never holds more than 3
    assert sched.add_request(a)
    most = 0
    while sched.has_work():
        run_step(sched)
        if a.status != RequestStatus.FINISHED:
            most = max(most, sum(p >= 0 for p in cache.table(0, a)))
    assert a.status == RequestStatus.FINISHED and most <= 3
