"""The scheduler's decisions, driven with a fake model that always answers token 77 (no GPU)."""

import pytest

from turboserve_b200.cache import CacheManager, GroupSpec
from turboserve_b200.config import FinishReason, SamplingParams, SchedulerConfig
from turboserve_b200.engine.scheduler import Scheduler, SchedulerOutput
from turboserve_b200.engine.sequence import SeqStatus


def make(pages=16, page_size=4, budget=16, seqs=4, window=None, chunked=True):
    groups = [GroupSpec("full", None, pages, page_size)]
    if window:
        groups.append(GroupSpec("w", window, pages, page_size))
    config = SchedulerConfig(max_num_seqs=seqs, max_num_batched_tokens=budget, block_size=page_size,
                             enable_chunked_prefill=chunked)
    return Scheduler(config, CacheManager(groups, seqs))


def run_step(s, token=77, eos=()):
    """One schedule + fake forward + sampling; returns the plan."""
    plan = s.schedule(now=0.0)
    s.check_invariants()
    seen = set()
    for item in plan.scheduled:
        assert item.seq.seq_id not in seen  # a request appears at most once in a step
        seen.add(item.seq.seq_id)
        assert len(item.token_ids) == item.num_new_tokens
        assert item.token_ids == item.seq.token_ids[item.start:item.start + item.num_new_tokens]
        for table, group in zip(item.block_tables, s.cache.groups):
            assert len(table) == -(-item.context_len // group.page_size)
    assert plan.num_tokens <= s.config.max_num_batched_tokens
    assert len(plan.scheduled) <= s.config.max_num_seqs
    kinds = [i.is_prefill for i in plan.scheduled]
    assert kinds == sorted(kinds, reverse=True)  # prefills, then decodes
    lengths = [i.context_len for i in plan.scheduled if not i.is_prefill]
    assert lengths == sorted(lengths, reverse=True)  # among the decodes the longest context first
    for item in plan.scheduled:
        if item.samples:
            s.append_token(item.seq, token, eos, now=0.0)
    s.check_invariants()
    return plan


def test_whole_prompt_then_decode_then_length():
    s = make()
    seq = s.add_request("a", list(range(10)), SamplingParams(max_tokens=3))
    plan = run_step(s)
    assert [(i.num_new_tokens, i.is_prefill, i.samples) for i in plan.scheduled] == [(10, True, True)]
    assert plan.admitted == [seq] and seq.output_token_ids == [77]
    plan = run_step(s)
    assert [(i.start, i.num_new_tokens, i.is_prefill) for i in plan.scheduled] == [(10, 1, False)]
    run_step(s)
    assert seq.is_finished and seq.finish_reason is FinishReason.LENGTH and seq.num_output_tokens == 3
    assert not s.has_unfinished() and s.cache.free_pages() == [16]


def test_prompt_is_cut_under_the_token_budget_and_samples_once():
    s = make(budget=8)
    seq = s.add_request("a", list(range(19)), SamplingParams(max_tokens=2))
    sizes = []
    while seq.num_output_tokens == 0:
        plan = run_step(s)
        sizes.append([(i.num_new_tokens, i.samples) for i in plan.scheduled])
    assert sizes == [[(8, False)], [(8, False)], [(3, True)]]


def test_decodes_go_first_and_a_new_prompt_gets_the_rest_of_the_budget():
    s = make(budget=8, pages=32)
    a = s.add_request("a", [1, 2, 3], SamplingParams(max_tokens=8))
    run_step(s)
    b = s.add_request("b", list(range(20)), SamplingParams(max_tokens=8))
    plan = run_step(s)
    assert [(i.seq.request_id, i.num_new_tokens, i.is_prefill) for i in plan.scheduled] == [("b", 7, True), ("a", 1, False)]
    plan = run_step(s)
    assert [(i.seq.request_id, i.num_new_tokens) for i in plan.scheduled] == [("b", 7), ("a", 1)]
    assert a.num_output_tokens == 3 and b.num_output_tokens == 0


def test_sequence_budget_and_queue_order():
    s = make(seqs=2, pages=32)
    for name in "abc":
        s.add_request(name, [1, 2, 3], SamplingParams(max_tokens=2))
    plan = run_step(s)
    assert [i.seq.request_id for i in plan.scheduled] == ["a", "b"]
    plan = run_step(s)  # a and b finish here (max_tokens=2), c still waits for a slot in this step
    assert [i.seq.request_id for i in plan.scheduled] == ["a", "b"]
    plan = run_step(s)
    assert [i.seq.request_id for i in plan.scheduled] == ["c"]


def test_no_chunking_waits_for_a_step_that_fits():
    s = make(budget=8, chunked=False)
    with pytest.raises(ValueError, match="chunked prefill is disabled"):
        s.add_request("big", list(range(9)))
    a = s.add_request("a", list(range(6)), SamplingParams(max_tokens=4))
    s.add_request("b", list(range(6)), SamplingParams(max_tokens=4))
    plan = run_step(s)
    assert [i.seq.request_id for i in plan.scheduled] == ["a"]  # b does not fit beside a and may not be split
    plan = run_step(s)
    assert sorted(i.seq.request_id for i in plan.scheduled) == ["a", "b"]
    assert a.num_output_tokens == 2


def test_requests_are_rejected_that_can_never_run():
    s = make(pages=2, page_size=4)
    with pytest.raises(ValueError, match="empty prompt"):
        s.add_request("e", [])
    with pytest.raises(ValueError, match="more than the cache can ever hold"):
        s.add_request("big", list(range(9)))
    s.add_request("a", [1])
    with pytest.raises(ValueError, match="already in flight"):
        s.add_request("a", [1])


def test_pages_run_out_the_newest_request_is_preempted_and_recomputed():
    s = make(pages=4, page_size=4, budget=16)
    a = s.add_request("a", list(range(7)), SamplingParams(max_tokens=6))
    b = s.add_request("b", list(range(100, 107)), SamplingParams(max_tokens=20))
    run_step(s)  # both prefill: 2 pages each, pool empty
    assert s.cache.free_pages() == [0]
    plan = run_step(s)  # position 7 still fits the second page of each
    assert len(plan.scheduled) == 2 and not plan.preempted
    plan = run_step(s)  # a needs a third page: b, admitted last, gives up everything
    assert plan.preempted == [b] and [i.seq.request_id for i in plan.scheduled] == ["a"]
    assert b.status is SeqStatus.PREEMPTED and b.num_computed_tokens == 0 and b.num_output_tokens == 2
    assert "b" not in s.cache and b.timing.num_preemptions == 1
    # b comes back only when its whole sequence (9 tokens -> 3 pages) fits again: after a ends
    steps = 0
    while not a.is_finished:
        plan = run_step(s)
        assert "b" not in [i.seq.request_id for i in plan.scheduled]
        steps += 1
    assert a.finish_reason is FinishReason.LENGTH and steps == 3 and s.cache.free_pages() == [4]
    plan = run_step(s)
    assert [(i.seq.request_id, i.start, i.num_new_tokens, i.is_prefill, i.samples) for i in plan.scheduled] == [("b", 0, 9, True, True)]
    assert b.token_ids[:9] == list(range(100, 107)) + [77, 77]  # outputs so far are kept and recomputed


def test_a_request_that_outgrows_the_whole_pool_is_ended_not_preempted_for_ever():
    s = make(pages=2, page_size=4)
    a = s.add_request("a", list(range(6)), SamplingParams(max_tokens=50))
    dropped = []
    for _ in range(20):
        plan = run_step(s)
        dropped += plan.dropped
        if not s.has_unfinished():
            break
    assert dropped == [a] and a.finish_reason is FinishReason.LENGTH
    assert a.num_tokens == 9  # 8 tokens fit two pages; the ninth was sampled but can never be computed
    assert s.cache.free_pages() == [2] and s.num_preemptions == 1


def test_recompute_cut_by_the_budget_samples_only_at_its_end():
    # The reference samples from the middle of a resumed request's history when the cut falls
    # after the prompt (its scheduler.py:728-738); here only the last portion samples.
    s = make(pages=8, page_size=4, budget=8)
    a = s.add_request("a", list(range(5)), SamplingParams(max_tokens=30))
    for _ in range(7):
        run_step(s)
    assert a.num_tokens == 12
    s._send_back(a, set(), SchedulerOutput())
    assert a.num_computed_tokens == 0 and a.num_tokens == 12
    plan = run_step(s)
    assert [(i.start, i.num_new_tokens, i.samples) for i in plan.scheduled] == [(0, 8, False)]
    assert a.num_tokens == 12  # nothing was sampled from the middle
    plan = run_step(s)
    assert [(i.start, i.num_new_tokens, i.samples, i.is_prefill) for i in plan.scheduled] == [(8, 4, True, False)]
    assert a.num_tokens == 13


def test_stop_tokens_eos_and_abort():
    s = make()
    a = s.add_request("a", [1, 2], SamplingParams(max_tokens=9, stop_token_ids=[77]))
    b = s.add_request("b", [1, 2], SamplingParams(max_tokens=9))
    c = s.add_request("c", [1, 2], SamplingParams(max_tokens=9, ignore_eos=True))
    run_step(s, token=77, eos=(77,))
    assert a.finish_reason is FinishReason.STOP and a.stop_token_id == 77
    assert b.finish_reason is FinishReason.STOP and not c.is_finished
    assert s.abort("c") and c.finish_reason is FinishReason.ABORT and not s.abort("c")
    assert not s.has_unfinished() and s.cache.free_pages() == [16] and s.cache.slots.num_free == 4


def test_schedule_is_deterministic():
    def trace():
        s = make(pages=6, page_size=4, budget=8, seqs=3)
        out = []
        for i, n in enumerate([9, 3, 14, 5]):
            s.add_request(f"r{i}", list(range(n)), SamplingParams(max_tokens=6))
        for _ in range(60):
            if not s.has_unfinished():
                break
            plan = run_step(s)
            out.append([(i.seq.request_id, i.start, i.num_new_tokens, i.samples) for i in plan.scheduled]
                       + [("preempted", [p.request_id for p in plan.preempted])])
        assert not s.has_unfinished()
        return out, s.stats()
    assert trace() == trace()


def test_windowed_group_lets_long_requests_run_in_few_pages():
    s = make(pages=8, page_size=4, budget=8, window=4)
    a = s.add_request("a", list(range(20)), SamplingParams(max_tokens=10))
    while s.has_unfinished():
        plan = run_step(s)
        if "a" in s.cache:
            assert sum(1 for p in s.cache.tables("a")[1] if p >= 0) <= 4
    assert a.finish_reason is FinishReason.LENGTH and s.cache.num_window_releases > 0
    assert s.cache.free_pages() == [8, 8]


def test_a_decode_step_is_planned_ahead_only_when_it_is_certain():
    """continue_decode: the step after a plan, before that plan's tokens are known."""
    s = make(pages=10, page_size=4, budget=16, seqs=4)
    a = s.add_request("a", [1, 2, 3], SamplingParams(max_tokens=20))
    b = s.add_request("b", [4, 5, 6, 7, 8], SamplingParams(max_tokens=20))
    plan = s.schedule(now=0.0)  # both prompts whole; both sample
    assert all(i.samples for i in plan.scheduled)
    ahead = s.continue_decode(plan)
    assert ahead is not None and [i.seq for i in ahead.scheduled] == [i.seq for i in plan.scheduled]
    # one token on, at the position of the token that is still to come; pages grown; ids are placeholders
    assert [(i.start, i.num_new_tokens, i.samples, i.is_prefill) for i in ahead.scheduled] == [(3, 1, True, False), (5, 1, True, False)]
    assert s.cache.num_tokens("a") == 4 and s.cache.num_tokens("b") == 6 and len(s.cache.tables("b")[0]) == 2
    for item in plan.scheduled:  # the tokens of the first plan arrive
        s.append_token(item.seq, 77, now=0.0)
    s.check_invariants()
    assert a.num_computed_tokens == a.num_tokens == 4
    # the next one again, then the tokens of `ahead`
    ahead2 = s.continue_decode(ahead)
    assert ahead2 is not None and [i.start for i in ahead2.scheduled] == [4, 6]
    for item in ahead.scheduled:
        s.append_token(item.seq, 78, now=0.0)
    s.check_invariants()
    assert a.output_token_ids == [77, 78]

    # somebody waits: the next step is the scheduler's to decide
    s.add_request("c", [9] * 3, SamplingParams(max_tokens=4))
    assert s.continue_decode(ahead2) is None
    for item in ahead2.scheduled:
        s.append_token(item.seq, 79, now=0.0)
    plan = run_step(s)  # admits c beside the two decodes
    assert sorted(i.seq.request_id for i in plan.scheduled) == ["a", "b", "c"]

    # a request that ended with the token before is still in the plan that was made ahead; the
    # plan after that is not made ahead, since the running set has changed
    plan = s.schedule(now=0.0)
    ahead = s.continue_decode(plan)
    assert ahead is not None
    for item in plan.scheduled:
        s.append_token(item.seq, 5 if item.seq is b else 80, eos_token_ids=(5,), now=0.0)
    assert b.is_finished and "b" not in s.cache
    assert s.continue_decode(ahead) is None
    s.check_invariants()


def test_no_plan_ahead_without_pages_or_for_a_prompt_that_is_cut():
    s = make(pages=2, page_size=4, budget=16, seqs=2)
    a = s.add_request("a", [1, 2, 3, 4], SamplingParams(max_tokens=20))
    b = s.add_request("b", [5, 6, 7, 8], SamplingParams(max_tokens=20))
    plan = s.schedule(now=0.0)  # both pages are taken; the next token of either needs a third
    assert len(plan.scheduled) == 2 and s.cache.free_pages() == [0]
    assert s.continue_decode(plan) is None
    assert s.cache.num_tokens("a") == 4 and a.num_computed_tokens == 4  # nothing was touched
    s = make(budget=4)
    s.add_request("a", list(range(10)), SamplingParams(max_tokens=4))
    plan = s.schedule(now=0.0)  # a portion of the prompt: it does not sample
    assert not plan.scheduled[0].samples and s.continue_decode(plan) is None
    assert s.continue_decode(SchedulerOutput()) is None


def test_a_windowed_group_with_exactly_the_pages_admission_asks_for_runs_and_one_fewer_is_refused():
    """A token budget far above the window: a portion needs the window before it plus itself.

    Window 32, pages of 8, portions of 251 tokens: the third portion starts at position 502, reads
    from position 471 (the last slot of page 58) and writes up to 752 (page 94): 37 pages at once,
    which is what ``pages_to_admit`` gives (36 for the 283 positions, one for the ragged start).
    With 37 pages the request runs to its end; with 36 it is refused when it is added; and a
    manager that is driven past that check does run out at that very portion.
    """
    from turboserve_b200.cache.manager import OutOfPagesError

    def make_windowed(pages):
        groups = [GroupSpec("full", None, 200, 8), GroupSpec("w", 32, pages, 8)]
        config = SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=251, block_size=8)
        return Scheduler(config, CacheManager(groups, 2))

    s = make_windowed(37)
    assert s.cache.pages_to_admit(760, 251) == [95, 37]
    seq = s.add_request("a", list(range(760)), SamplingParams(max_tokens=6))
    least_free = 37
    portions = []
    while s.has_unfinished():
        plan = run_step(s)
        portions += [(i.start, i.num_new_tokens) for i in plan.scheduled]
        least_free = min(least_free, s.cache.free_pages()[1])
        assert not plan.preempted and not plan.dropped
    assert portions[:4] == [(0, 251), (251, 251), (502, 251), (753, 7)] and seq.num_output_tokens == 6
    assert least_free == 0  # every page of the group was in use at the third portion
    with pytest.raises(ValueError, match="more than the cache can ever hold"):
        make_windowed(36).add_request("a", list(range(760)), SamplingParams(max_tokens=6))
    manager = CacheManager([GroupSpec("w", 32, 36, 8)], 1)
    manager.admit("a")
    manager.grow("a", 251)
    manager.grow("a", 251)
    with pytest.raises(OutOfPagesError):
        manager.grow("a", 251)
