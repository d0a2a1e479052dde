"""The scheduler's decisions on the CPU, with the model replaced by a stand-in that stores tokens and returns
a fixed next token: admission order, token budget, portions, decode, finish, and what happens when pages run out."""
from __future__ import annotations

import pytest

from cuinfer_b200.cache import CacheGroupSpec, CacheManager
from cuinfer_b200.engine.scheduler import FinishReason, RequestStatus, Scheduler
from cuinfer_b200.sampling import SamplingParams


def make(num_pages, page_size=16, budget=24, max_seqs=8, max_len=256, eos=()):
    mgr = CacheManager([CacheGroupSpec((0,), 2, 16, None)], page_size, num_pages, max_seqs)
    return mgr, Scheduler(mgr, max_num_seqs=max_seqs, max_num_scheduled_tokens=budget, max_model_len=max_len,
                          eos_token_ids=eos)


def run_step(mgr, sched, next_token=lambda req: 100):
    """What the engine does around the scheduler: run the scheduled tokens (here: record them), sample, update."""
    scheduled = sched.schedule()
    for s in scheduled:
        assert mgr.num_tokens(s.request.request_id) == s.position_offset
        mgr.commit(s.request.request_id, len(s.tokens))
    mgr.check()
    sampled = [(s.request.request_id, next_token(s.request)) for s in scheduled if s.needs_sampling]
    return scheduled, sched.update(sampled)


def shape(scheduled):
    return [(s.request.request_id, s.position_offset, len(s.tokens), s.needs_sampling) for s in scheduled]


def test_budget_cuts_prompts_into_portions_beside_decodes():
    mgr, sched = make(num_pages=6, budget=24)
    p = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    sched.add_request("a", list(range(5)), p)
    sched.add_request("b", list(range(17)), p)
    sched.add_request("c", list(range(33)), p)
    s1, _ = run_step(mgr, sched)
    assert shape(s1) == [("a", 0, 5, True), ("b", 0, 17, True), ("c", 0, 2, False)]     # c cut by the budget
    s2, _ = run_step(mgr, sched)
    assert shape(s2) == [("a", 5, 1, True), ("b", 17, 1, True), ("c", 2, 22, False)]    # decodes beside a portion
    s3, _ = run_step(mgr, sched)
    assert shape(s3) == [("a", 6, 1, True), ("b", 18, 1, True), ("c", 24, 9, True)]     # the portion that ends the prompt samples
    assert all(not s.is_prefill for s in s3[:2]) and s3[2].is_prefill


def test_finish_by_length_eos_and_model_len():
    mgr, sched = make(num_pages=16, eos=(7,), max_len=12)
    sched.add_request("len", [1, 2, 3], SamplingParams(max_tokens=2))
    sched.add_request("eos", [1, 2], SamplingParams(max_tokens=50))
    sched.add_request("ign", [1, 2], SamplingParams(max_tokens=3, ignore_eos=True))
    sched.add_request("max", list(range(10)), SamplingParams(max_tokens=50, ignore_eos=True))
    outs = []
    for _ in range(4):
        _, o = run_step(mgr, sched, next_token=lambda req: 7 if req.request_id in ("eos", "ign") else 5)
        outs += o
    by = {}
    for o in outs:
        by.setdefault(o.request_id, []).append(o)
    assert [o.finish_reason for o in by["len"]] == [FinishReason.RUNNING, FinishReason.LENGTH]
    assert [o.finish_reason for o in by["eos"]] == [FinishReason.STOP] and by["eos"][0].new_token_ids == [7]
    assert [o.finish_reason for o in by["ign"]] == [FinishReason.RUNNING, FinishReason.RUNNING, FinishReason.LENGTH]
    assert [o.finish_reason for o in by["max"]] == [FinishReason.RUNNING, FinishReason.LENGTH]   # 12 tokens = max_model_len
    assert not sched.has_requests() and mgr.num_free_pages() == 16 and not mgr.live_requests()


def test_pages_run_out_last_running_is_preempted_and_recomputed():
    mgr, sched = make(num_pages=4, budget=64)
    p = SamplingParams(max_tokens=40, ignore_eos=True)
    sched.add_request("a", list(range(30)), SamplingParams(max_tokens=6, ignore_eos=True))   # 2 pages
    sched.add_request("b", list(range(31)), p)          # 2 pages -> pool full
    s1, _ = run_step(mgr, sched)
    assert shape(s1) == [("a", 0, 30, True), ("b", 0, 31, True)]
    s2, _ = run_step(mgr, sched)                         # a: 31 tokens fits; b: 32 fits
    assert shape(s2) == [("a", 30, 1, True), ("b", 31, 1, True)]
    s3, _ = run_step(mgr, sched)                         # a needs a third page: none free -> b (last) is preempted
    assert shape(s3) == [("a", 31, 1, True)]
    b = sched.requests["b"]
    assert b.status == RequestStatus.PREEMPTED and b.num_computed_tokens == 0 and "b" not in mgr
    assert sched.num_preemptions == 1
    # b waits while a holds 3 of 4 pages; when a finishes, b recomputes prompt + its 2 outputs as one prefill
    steps = 0
    while "a" in sched.requests:
        s, _ = run_step(mgr, sched)
        assert [x[0] for x in shape(s)] == ["a"]
        steps += 1
    s, _ = run_step(mgr, sched)
    assert shape(s) == [("b", 0, 33, True)] and s[0].is_prefill
    assert sched.requests["b"].num_output_tokens == 3


def test_victim_is_the_request_itself_when_it_is_last():
    mgr, sched = make(num_pages=3, budget=64)
    p = SamplingParams(max_tokens=40, ignore_eos=True)
    sched.add_request("a", list(range(16)), p)
    sched.add_request("b", list(range(32)), p)
    run_step(mgr, sched)                                 # a: 1 page, b: 2 pages
    s2, _ = run_step(mgr, sched)                         # a needs page 2 -> preempts b; then a fits
    assert shape(s2) == [("a", 16, 1, True)]
    assert sched.requests["b"].status == RequestStatus.PREEMPTED
    s3, _ = run_step(mgr, sched)                         # b cannot come back: 1 page free, needs 3
    assert shape(s3) == [("a", 17, 1, True)]


def test_a_request_alone_that_cannot_fit_finishes_with_capacity():
    mgr, sched = make(num_pages=2, budget=64)
    sched.add_request("a", list(range(30)), SamplingParams(max_tokens=40, ignore_eos=True))
    outs = []
    for _ in range(8):
        _, o = run_step(mgr, sched)
        outs += o
        if not sched.has_requests():
            break
    assert outs[-1].finish_reason == FinishReason.CAPACITY and outs[-1].new_token_ids == []
    assert sum(len(o.new_token_ids) for o in outs) == 3          # 30 + 3 = 33 tokens would need a third page
    assert mgr.num_free_pages() == 2 and not sched.has_requests()
    with pytest.raises(ValueError, match="cannot fit"):
        sched.add_request("big", list(range(40)), SamplingParams())


def test_admission_order_and_seq_limit_and_abort():
    mgr, sched = make(num_pages=32, budget=100, max_seqs=2)
    p = SamplingParams(max_tokens=3, ignore_eos=True)
    for name in "abcd":
        sched.add_request(name, [1, 2, 3], p)
    with pytest.raises(ValueError, match="already"):
        sched.add_request("a", [1], p)
    s1, _ = run_step(mgr, sched)
    assert [x[0] for x in shape(s1)] == ["a", "b"]               # max_num_seqs
    sched.abort_requests(["b", "zzz"])
    assert "b" not in mgr and "b" not in sched.requests
    s2, _ = run_step(mgr, sched)
    assert [x[0] for x in shape(s2)] == ["a", "c"]               # first come, first served
    sched.abort_requests(["d"])                                  # abort while waiting
    while sched.has_requests():
        run_step(mgr, sched)
    assert mgr.num_free_pages() == 32


def test_no_admission_in_a_step_that_preempted():
    mgr, sched = make(num_pages=2, budget=64)
    p = SamplingParams(max_tokens=40, ignore_eos=True)
    sched.add_request("a", list(range(16)), p)
    sched.add_request("b", list(range(16)), p)
    run_step(mgr, sched)
    sched.add_request("c", [1], p)
    s2, _ = run_step(mgr, sched)        # a needs a page -> b preempted; c (waiting) is not admitted in this step
    assert shape(s2) == [("a", 16, 1, True)]
    assert sched.requests["c"].status == RequestStatus.WAITING
