"""The scheduler's decisions, driven with a fake forward (every sampled token is given by
the test), as the reference tests its scheduler with a zero-layer model
(tests/engine_step.rs, tests/cache_scheduler_plan.rs, tests/prefix_cache.rs)."""
import random

import pytest

from vosti_b200.cache import CacheManager
from vosti_b200.engine import AdmissionStatus, Request, Scheduler, SchedulerConfig
from vosti_b200.parts import PagedCacheSpec

SPEC = PagedCacheSpec(2, 2, 16)


def make(num_pages=16, page_size=4, max_num_seqs=4, budget=64, chunk=0, slots=None, reuse=True, **kw):
    cache = CacheManager([SPEC], [None], num_pages=num_pages, page_size=page_size,
                         max_requests=slots or max_num_seqs, prefix_reuse=reuse)
    return cache, Scheduler(cache, SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=budget,
                                                  prefill_chunk_size=chunk, **kw))


def run_step(cache, sched, token=lambda row: 1):
    """What the engine does around a forward: reserve the rows' cache entries, then commit."""
    plan = sched.plan()
    for row in plan.rows:
        assert row.start == cache.length(row.request.request_id)
        cache.extend(row.request.request_id, row.count)
    emitted = sched.commit(plan, [token(r) if r.sample else None for r in plan.rows])
    cache.check()
    return plan, emitted


def rows(plan):
    return [(r.request.request_id, r.start, r.count, r.sample) for r in plan.rows]


def test_admission_checks():
    _, sched = make(vocab_size=100, max_context=32)
    ok = Request(1, [1, 2, 3], 4, eos_token_ids=(0,))
    assert sched.add_request(ok) is AdmissionStatus.ACCEPTED
    assert sched.add_request(Request(1, [1], 4, eos_token_ids=(0,))) is AdmissionStatus.DUPLICATE_ID
    assert sched.add_request(Request(2, [], 4, eos_token_ids=(0,))) is AdmissionStatus.EMPTY_PROMPT
    assert sched.add_request(Request(3, [1], 0, eos_token_ids=(0,))) is AdmissionStatus.ZERO_BUDGET
    assert sched.add_request(Request(4, [1], 4, eos_token_ids=())) is AdmissionStatus.BAD_EOS
    assert sched.add_request(Request(5, [1], 4, eos_token_ids=(1, 2, 3, 4))) is AdmissionStatus.BAD_EOS
    assert sched.add_request(Request(6, [1] * 30, 4, eos_token_ids=(0,))) is AdmissionStatus.TOO_LONG
    assert sched.add_request(Request(7, [100], 4, eos_token_ids=(0,))) is AdmissionStatus.BAD_TOKEN
    assert sched.add_request(Request(8, [1], 4, eos_token_ids=(0,), temperature=-1.0)) is AdmissionStatus.BAD_SAMPLING
    assert sched.add_request(Request(9, [1], 4, ignore_eos=True)) is AdmissionStatus.ACCEPTED
    assert [r.request_id for r in sched.waiting] == [1, 9]


def test_no_pages_are_taken_before_the_first_plan():
    cache, sched = make()
    sched.add_request(Request(0, list(range(10)), 2, ignore_eos=True))
    assert cache.available_pages() == 16 and not cache.live
    run_step(cache, sched)
    assert cache.length(0) == 10


def test_whole_prompt_then_decode_until_max_tokens():
    cache, sched = make()
    sched.add_request(Request(0, list(range(10)), 3, ignore_eos=True))
    plan, emitted = run_step(cache, sched, lambda r: 41)
    assert rows(plan) == [(0, 0, 10, True)] and emitted == {0: 41}
    plan, _ = run_step(cache, sched, lambda r: 42)
    assert rows(plan) == [(0, 10, 1, True)]
    plan, emitted = run_step(cache, sched, lambda r: 43)
    assert rows(plan) == [(0, 11, 1, True)] and emitted == {0: 43}
    assert not sched.has_unfinished() and sched.finished[0].generated == [41, 42, 43]
    assert sched.finished[0].finish_reason == "length" and cache.available_pages() == 16


def test_eos_finishes_unless_ignored():
    cache, sched = make()
    sched.add_request(Request(0, [5, 6], 10, eos_token_ids=(9, 11)))
    sched.add_request(Request(1, [5, 7], 3, eos_token_ids=(9,), ignore_eos=True))
    run_step(cache, sched, lambda r: 11)
    assert sched.finished[0].finish_reason == "eos" and 1 not in sched.finished
    while sched.has_unfinished():
        run_step(cache, sched, lambda r: 9)
    assert sched.finished[1].generated == [11, 9, 9]


def test_prompt_is_cut_into_whole_pages_and_only_the_last_portion_samples():
    cache, sched = make(budget=10, reuse=False)
    sched.add_request(Request(0, list(range(23)), 2, ignore_eos=True))
    plan, emitted = run_step(cache, sched)
    assert rows(plan) == [(0, 0, 8, False)] and emitted == {}        # 10 // 4 * 4
    plan, _ = run_step(cache, sched)
    assert rows(plan) == [(0, 8, 8, False)]
    plan, emitted = run_step(cache, sched)
    assert rows(plan) == [(0, 16, 7, True)] and 0 in emitted
    assert len(cache.block_row(0, 0)) == 6


def test_explicit_chunk_size_beside_decodes():
    cache, sched = make(num_pages=64, page_size=8, budget=64, chunk=8, reuse=False)
    sched.add_request(Request(0, list(range(9)), 8, ignore_eos=True))
    run_step(cache, sched)
    plan, _ = run_step(cache, sched)
    assert rows(plan) == [(0, 8, 1, True)]
    sched.add_request(Request(1, list(range(40)), 2, ignore_eos=True))
    plan, _ = run_step(cache, sched)
    assert rows(plan) == [(0, 9, 1, True), (1, 0, 8, False)]          # a decode row beside a portion
    for start in (8, 16, 24):
        plan, _ = run_step(cache, sched)
        assert rows(plan)[1] == (1, start, 8, False)
    plan, _ = run_step(cache, sched)
    assert rows(plan)[1] == (1, 32, 8, True)


def test_decode_rows_use_up_the_budget_but_are_not_limited_by_it():
    cache, sched = make(num_pages=64, max_num_seqs=4, budget=6, reuse=False)
    for i in range(3):
        sched.add_request(Request(i, [i + 1] * 2, 4, ignore_eos=True))
    plan, _ = run_step(cache, sched)
    assert [r[0] for r in rows(plan)] == [0, 1, 2]
    sched.add_request(Request(3, [7] * 9, 2, ignore_eos=True))
    plan, _ = run_step(cache, sched)
    assert rows(plan) == [(0, 2, 1, True), (1, 2, 1, True), (2, 2, 1, True)]   # 3 left of the budget: no whole page
    assert [r.request_id for r in sched.waiting] == [3]


def test_head_of_line_blocking_and_fifo():
    cache, sched = make(num_pages=6, budget=64, reuse=False)
    sched.add_request(Request(0, [1] * 12, 2, ignore_eos=True))      # 3 pages
    sched.add_request(Request(1, [2] * 16, 2, ignore_eos=True))      # 4 pages: does not fit beside 0
    sched.add_request(Request(2, [3] * 2, 2, ignore_eos=True))       # would fit, but waits behind 1
    plan, _ = run_step(cache, sched)
    assert [r[0] for r in rows(plan)] == [0]
    assert [r.request_id for r in sched.waiting] == [1, 2]
    while 0 not in sched.finished:
        plan, _ = run_step(cache, sched)
    plan, _ = run_step(cache, sched)
    assert [r[0] for r in rows(plan)][:1] == [1]


def test_max_num_seqs_limits_rows():
    cache, sched = make(num_pages=64, max_num_seqs=2, slots=4, reuse=False)
    for i in range(4):
        sched.add_request(Request(i, [i + 1] * 3, 2, ignore_eos=True))
    plan, _ = run_step(cache, sched)
    assert [r[0] for r in rows(plan)] == [0, 1]
    plan, _ = run_step(cache, sched)
    assert [r[0] for r in rows(plan)] == [0, 1]                      # both finish here (2 tokens)
    plan, _ = run_step(cache, sched)
    assert [r[0] for r in rows(plan)] == [2, 3]


def test_prefix_reuse_only_from_earlier_steps():
    cache, sched = make(num_pages=32, budget=256)
    shared = list(range(50, 62))                                      # three pages
    sched.add_request(Request(0, shared + [1, 2], 2, ignore_eos=True))
    sched.add_request(Request(1, shared + [3, 4], 2, ignore_eos=True))
    plan, _ = run_step(cache, sched)
    # both are computed in the same step: the second cannot read pages the first is still producing
    assert rows(plan) == [(0, 0, 14, True), (1, 0, 14, True)]
    sched.add_request(Request(2, shared + [5, 6, 7], 2, ignore_eos=True))
    plan, _ = run_step(cache, sched)
    assert rows(plan)[-1] == (2, 12, 3, True)                         # three pages found again
    assert cache.requests_with_reuse == 1 and cache.reused_prefix_pages == 3


def test_pages_run_out_youngest_is_preempted_and_recomputed():
    cache, sched = make(num_pages=8, page_size=4, max_num_seqs=3, budget=64)
    for i in range(3):
        sched.add_request(Request(i, [10 * i + k for k in range(8)], 12, ignore_eos=True))
    seen_preempted = []
    steps = 0
    while sched.has_unfinished():
        plan, _ = run_step(cache, sched, lambda r: 100 + r.request.request_id)
        assert plan.rows, "a live request always makes progress"
        seen_preempted += plan.preempted
        steps += 1
        assert steps < 200
    assert seen_preempted and sched.preemptions == len(seen_preempted)
    assert 0 not in seen_preempted                                    # the oldest is never the victim here
    for i in range(3):
        assert sched.finished[i].generated == [100 + i] * 12         # preemption loses no token
    assert cache.available_pages() == 8


def test_request_too_large_for_any_cache_is_dropped():
    cache, sched = make(num_pages=4, page_size=4, budget=64, reuse=False)
    sched.add_request(Request(0, [1] * 40, 2, ignore_eos=True))
    sched.add_request(Request(1, [2] * 5, 2, ignore_eos=True))
    plan, _ = run_step(cache, sched)
    assert plan.dropped == [0] and sched.finished[0].finish_reason == "capacity"
    assert [r[0] for r in rows(plan)] == [1]


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_with_every_token(seed):
    rng = random.Random(seed)
    cache, sched = make(num_pages=rng.choice([6, 10, 24]), page_size=rng.choice([2, 4, 8]),
                        max_num_seqs=rng.choice([1, 2, 4]), budget=rng.choice([8, 16, 64]),
                        chunk=rng.choice([0, 8]), reuse=bool(seed % 2))
    total_pages = cache.num_pages
    want, arrivals = {}, []
    for i in range(10):
        prompt = [rng.randrange(5) for _ in range(rng.randrange(1, 14))]
        max_tokens = rng.randrange(1, 7)
        if cache.pages_for(len(prompt) + max_tokens) <= total_pages:
            want[i] = max_tokens
        arrivals.append((rng.randrange(0, 20), Request(i, prompt, max_tokens, ignore_eos=True)))
    step = 0
    while arrivals or sched.has_unfinished():
        for item in [a for a in arrivals if a[0] <= step]:
            arrivals.remove(item)
            assert sched.add_request(item[1]) is AdmissionStatus.ACCEPTED
        if sched.has_unfinished():
            plan, _ = run_step(cache, sched, lambda r: len(r.request.generated))
            assert plan.rows or plan.dropped
            assert len(plan.rows) <= sched.config.max_num_seqs
            prefill = sum(r.count for r in plan.rows if r.count > 1)
            assert prefill <= sched.config.max_num_batched_tokens
        step += 1
        assert step < 2000
    for rid, n in want.items():
        assert sched.finished[rid].generated == list(range(n))
    assert cache.available_pages() == total_pages and not cache.live


def test_abort_gives_everything_back():
    cache, sched = make(num_pages=16)
    sched.add_request(Request(0, [1] * 9, 5, ignore_eos=True))
    sched.add_request(Request(1, [2] * 9, 5, ignore_eos=True))
    run_step(cache, sched)
    assert sched.abort(0) and not sched.abort(0) and not sched.abort(77)
    assert [r.request_id for r in sched.running] == [1] and sched.finished[0].finish_reason == "aborted"
    cache.check()
    while sched.has_unfinished():
        run_step(cache, sched)
    assert cache.available_pages() == 16


def _token(rid, index):
    """What the "model" samples: a function of the request and the place only."""
    return (rid * 31 + index * 7) % 11


def _workload(rng, cache):
    arrivals = []
    for i in range(10):
        prompt = [rng.randrange(5) for _ in range(rng.randrange(1, 14))]
        max_tokens = rng.randrange(1, 9)
        eos = (rng.randrange(11),) if i % 2 else ()
        if cache.pages_for(len(prompt) + max_tokens) <= cache.num_pages:
            arrivals.append((rng.randrange(0, 20), i, prompt, max_tokens, eos))
    return arrivals


@pytest.mark.parametrize("seed", range(8))
def test_commit_in_two_halves_gives_the_tokens_of_the_plain_commit(seed):
    """commit_ahead, the next plan, then resolve (what the engine does when it launches a step
    before it has read the last one's tokens) give every request the tokens and the finish
    reason the plain commit gives: EOS, length limits, prefix reuse, and so few pages that
    requests are preempted while their newest token is still pending. No page is lost."""
    outcomes = []
    for ahead in (False, True):
        rng = random.Random(seed)
        cache, sched = make(num_pages=rng.choice([6, 10, 24]), page_size=rng.choice([2, 4, 8]),
                            max_num_seqs=rng.choice([1, 2, 4]), budget=rng.choice([8, 16, 64]),
                            chunk=rng.choice([0, 8]), reuse=bool(seed % 2))
        arrivals = _workload(rng, cache)
        ids = [a[1] for a in arrivals]
        sample = lambda plan: [_token(r.request.request_id, len(r.request.generated) - (1 if ahead else 0))
                               if r.sample else None for r in plan.rows]
        before, step = None, 0
        while arrivals or sched.has_unfinished() or before is not None:
            for item in [a for a in arrivals if a[0] <= step]:
                arrivals.remove(item)
                request = Request(item[1], item[2], item[3], item[4], ignore_eos=not item[4])
                assert sched.add_request(request) is AdmissionStatus.ACCEPTED
            if not ahead:
                if sched.has_unfinished():
                    plan = sched.plan()
                    for row in plan.rows:
                        cache.extend(row.request.request_id, row.count)
                    sched.commit(plan, sample(plan))
            else:
                if before is not None:
                    sched.commit_ahead(before)
                plan = sched.plan() if sched.has_unfinished() else None
                if plan is not None:
                    for row in plan.rows:
                        assert row.start == cache.length(row.request.request_id)
                        cache.extend(row.request.request_id, row.count)
                        tokens = row.request.token_range(row.start, row.count)
                        assert Scheduler.PENDING not in tokens[:-1]          # only the newest token can be pending
                if before is not None:
                    sched.resolve(before, sample(before))
                before = plan if plan is not None and plan.rows else None
            cache.check()
            step += 1
            assert step < 4000
        assert cache.available_pages() == cache.num_pages and not cache.live
        outcomes.append({rid: (sched.finished[rid].generated, sched.finished[rid].finish_reason) for rid in ids})
    assert outcomes[0] == outcomes[1]


def test_reuse_counters_do_not_count_a_blocked_admission_twice():
    """A waiting request whose prefix matches but which does not fit yet is tried every step;
    only its admission counts."""
    cache, sched = make(num_pages=8, page_size=4, max_num_seqs=2, budget=64)
    shared = [1, 2, 3, 4, 5, 6, 7, 8]
    sched.add_request(Request(0, shared + [9], 12, ignore_eos=True))
    run_step(cache, sched)
    sched.add_request(Request(1, shared + [3] * 23, 1, ignore_eos=True))      # needs more pages than are free
    for _ in range(4):
        plan, _ = run_step(cache, sched)
        assert [r.request.request_id for r in plan.rows] == [0]
    assert cache.requests_with_reuse == 0 and cache.reused_prefix_pages == 0
    while sched.has_unfinished():
        run_step(cache, sched)
    assert cache.requests_with_reuse == 1 and cache.reused_prefix_pages == 2


def test_a_step_cap_below_one_page_is_refused():
    """Prompts are cut into whole pages: with a per-step cap below the page size a long prompt
    could never be scheduled, so such settings are refused when the scheduler is made."""
    with pytest.raises(ValueError, match="less than one page"):
        make(num_pages=16, page_size=16, budget=64, chunk=8)
    with pytest.raises(ValueError, match="less than one page"):
        make(num_pages=16, page_size=16, budget=12)
    cache, sched = make(num_pages=16, page_size=16, budget=64, chunk=16)
    sched.add_request(Request(0, list(range(20)), 2, ignore_eos=True))
    plan, _ = run_step(cache, sched)
    assert rows(plan) == [(0, 0, 16, False)]
    plan, emitted = run_step(cache, sched)
    assert rows(plan) == [(0, 16, 4, True)] and 0 in emitted


@pytest.mark.parametrize("ahead", [False, True])
def test_host_records_do_not_grow_with_the_number_of_requests(ahead):
    """A finished request leaves nothing behind but its id and (for the newest few) its record."""
    import ctypes
    cache = CacheManager([SPEC], [None], num_pages=16, page_size=4, max_requests=2, prefix_reuse=True)
    sched = Scheduler(cache, SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=64, keep_finished=5))
    before = None
    for i in range(60):
        sched.add_request(Request(i, [i % 7, 3, 4, 5, 6], 2, eos_token_ids=(9,)))
        if i % 10 == 3:
            assert sched.abort(i)
        for _ in range(2):
            if not ahead:
                run_step(cache, sched, lambda r: 9 if r.request.request_id % 3 == 0 else 1)
                continue
            if before is not None:
                sched.commit_ahead(before)
            plan = sched.plan() if sched.has_unfinished() else None
            for row in (plan.rows if plan else []):
                cache.extend(row.request.request_id, row.count)
            if before is not None:
                sched.resolve(before, [(9 if r.request.request_id % 3 == 0 else 1) if r.sample else None
                                       for r in before.rows])
            before = plan if plan is not None and plan.rows else None
        assert len(sched._requests) <= 4 and len(cache._handles) <= 4 and len(cache._names) <= 4
        assert len(sched.finished) <= 5
    while sched.has_unfinished() or before is not None:
        if not ahead:
            run_step(cache, sched)
        else:
            sched.commit_ahead(before)
            sched.resolve(before, [1 if r.sample else None for r in before.rows])
            before = None
    assert not sched._requests and not cache._handles and not cache._names
    assert sched._lib.vh_request_field(sched._h, ctypes.c_int64(1), 0) < 0     # the core forgot it too
    assert sched.add_request(Request(0, [1], 1, ignore_eos=True)) is AdmissionStatus.DUPLICATE_ID
    assert sched.release(59) and not sched.release(59)
    cache.check()


def test_state_slots_handed_out_by_the_scheduler_are_reported_for_clearing():
    """A model with per-request state: every admission, by `begin` or inside the scheduler's
    plan, and every re-admission after a preemption, puts the slot on the list the step
    function clears before it runs."""
    import ctypes
    from vosti_b200 import host
    from vosti_b200.parts import StateSpec
    cache = CacheManager([SPEC], [StateSpec((4,))], num_pages=6, page_size=4, max_requests=2, prefix_reuse=True)
    assert cache.has_state and not cache.prefix_reuse
    sched = Scheduler(cache, SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=64))
    buf = (ctypes.c_int32 * 8)()
    take = lambda: sorted(buf[:cache._lib.vh_take_fresh_slots(cache._h, buf, 8)])
    assert take() == []
    for i in range(2):
        sched.add_request(Request(i, [1] * 8, 8, ignore_eos=True))
    plan, _ = run_step(cache, sched)
    first = {r.request.request_id: cache.slot(r.request.request_id) for r in plan.rows}
    assert take() == sorted(first.values()) and take() == []
    fresh, preempted = [], []
    while sched.has_unfinished():
        plan, _ = run_step(cache, sched)
        preempted += plan.preempted
        fresh += take()
    assert preempted and len(fresh) >= len(preempted)      # each re-admission was reported again
    sched.add_request(Request(7, [1] * 3, 1, ignore_eos=True))
    run_step(cache, sched)
    assert len(take()) == 1
