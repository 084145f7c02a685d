"""The scheduler's decisions with a fake model: decode first, budget split, one portion
per prompt per step, rotation, what happens when pages run out, finishing."""
import pytest

from tiny_llm_infer_b200.cache import CacheManager
from tiny_llm_infer_b200.engine.scheduler import (Scheduler, SchedulerConfig, SchedulerError, Sequence,
                                                  Status)
from tiny_llm_infer_b200.parts.spec import CacheSpec
from tiny_llm_infer_b200.sampling import SamplingParams

NEEDS = {0: (CacheSpec.keys_and_values(1, 16, None), None)}


def make(pages=16, budget=32, seqs=4, page=8):
    cache = CacheManager(NEEDS, page, pages, seqs, 256)
    return Scheduler(SchedulerConfig(seqs, budget, page, pages), cache), cache


def seq(i, n, max_tokens=4, **kw):
    return Sequence(i, list(range(n)), SamplingParams(max_tokens=max_tokens, ignore_eos=True, **kw))


def run_step(sched, cache, token=7, eos=()):
    """What the engine does around a step, with a model that always says ``token``."""
    plan = sched.schedule()
    for item in plan.sequences:                      # the step function's bookkeeping
        assert cache.computed(item.sequence.id) == item.token_start
        cache.reserve(item.sequence.id, item.token_start + item.token_count)
        cache.commit(item.sequence.id, item.token_start + item.token_count)
    sampled = [token if item.samples else -1 for item in plan.sequences]
    done = sched.postprocess(plan, sampled, lambda t: t in eos)
    cache.audit()
    return plan, done


def shape(plan):
    return [(s.sequence.id, s.token_start, s.token_count, s.is_prefill) for s in plan.sequences]


def test_prompts_are_cut_under_the_budget_and_rotate():
    sched, cache = make(pages=32, budget=32)
    for i, n in enumerate((40, 9, 70)):
        sched.add(seq(i + 1, n))
    plan, _ = run_step(sched, cache)
    assert shape(plan) == [(1, 0, 32, True)] and plan.num_tokens == 32 and plan.is_prefill
    plan, _ = run_step(sched, cache)                 # 1 went to the back: 2 and 3 come first
    assert shape(plan) == [(2, 0, 9, True), (3, 0, 23, True)]
    assert [s.samples for s in plan.sequences] == [True, False]
    plan, _ = run_step(sched, cache)                 # decode of 2 first, then portions
    assert shape(plan) == [(2, 9, 1, False), (1, 32, 8, True), (3, 23, 23, True)]
    assert not plan.is_prefill
    plan, _ = run_step(sched, cache)
    assert shape(plan) == [(2, 10, 1, False), (1, 40, 1, False), (3, 46, 24, True)]


def test_finishes_on_max_tokens_and_eos_and_frees():
    sched, cache = make()
    sched.add(seq(1, 5, max_tokens=2))
    s2 = Sequence(2, [1, 2, 3], SamplingParams(max_tokens=50))
    sched.add(s2)
    _, done = run_step(sched, cache, token=9)
    assert done == []
    _, done = run_step(sched, cache, token=9)
    assert [d.id for d in done] == [1] and done[0].completion == [9, 9] and done[0].status is Status.FINISHED
    _, done = run_step(sched, cache, token=3, eos={3})
    assert [d.id for d in done] == [2] and s2.completion == [9, 9, 3]
    assert sched.is_finished() and cache.free_pages() == {None: 16} and cache.free_slots == 4


def test_waiting_for_pages_without_preemption():
    sched, cache = make(pages=4, budget=64)
    sched.add(seq(1, 17, max_tokens=3))                # 3 pages
    sched.add(seq(2, 16, max_tokens=3))                # 2 pages, 3 when it grows: must wait
    plan, _ = run_step(sched, cache)
    assert shape(plan) == [(1, 0, 17, True)]
    steps = 1
    while not sched.is_finished():
        run_step(sched, cache)
        steps += 1
        assert steps < 20
    assert sched.num_preemptions == 0


def test_out_of_pages_preempts_the_oldest_that_cannot_grow_and_recomputes():
    sched, cache = make(pages=4, budget=64, page=8)
    a, b = seq(1, 15, max_tokens=6), seq(2, 15, max_tokens=6)
    sched.add(a), sched.add(b)
    run_step(sched, cache)                             # both prompts whole: 2 pages each
    plan, _ = run_step(sched, cache)                   # position 15 still fits their pages
    assert shape(plan) == [(1, 15, 1, False), (2, 15, 1, False)]
    plan, _ = run_step(sched, cache)                   # position 16 needs a third page: none free
    assert [s.id for s in plan.preempted] == [1] and sched.num_preemptions == 1
    assert shape(plan) == [(2, 16, 1, False)]          # 1 gave its pages back, 2 grows into them
    assert a.num_cached_tokens == 0 and a.status is Status.WAITING and len(a) == 17
    done_ids = []
    for _ in range(40):
        if sched.is_finished():
            break
        plan, done = run_step(sched, cache)
        done_ids += [d.id for d in done]
        for s in plan.sequences:
            if s.sequence is a and s.is_prefill:
                assert (s.token_start, s.token_count) == (0, 17)    # its prompt and its two generated tokens again
    assert sorted(done_ids) == [1, 2] and a.completion == [7] * 6 and b.completion == [7] * 6
    assert cache.free_pages() == {None: 4}


def test_prompt_larger_than_the_pool_is_an_error():
    sched, cache = make(pages=2, page=8)
    sched.add(seq(1, 17))
    with pytest.raises(SchedulerError, match="needs 3 pages, the pool has 2"):
        sched.schedule()


def test_slots_bound_live_requests():
    sched, cache = make(seqs=2, budget=64)
    for i in range(3):
        sched.add(seq(i + 1, 4, max_tokens=2))
    plan, _ = run_step(sched, cache)
    assert [s.sequence.id for s in plan.sequences] == [1, 2]
    run_step(sched, cache)
    plan, _ = run_step(sched, cache)
    assert 3 in [s.sequence.id for s in plan.sequences]


def test_empty_request_and_wrong_sample_count():
    sched, cache = make()
    with pytest.raises(ValueError):
        sched.add(Sequence(1, [], SamplingParams()))
    sched.add(seq(1, 3))
    plan = sched.schedule()
    with pytest.raises(SchedulerError, match="0 sampled tokens for a plan of 1"):
        sched.postprocess(plan, [], lambda t: False)


def test_prefix_cache_starts_a_prompt_behind_what_is_shared():
    """A prompt that begins like an earlier one is admitted with its full shared pages counted
    as computed (engine/src/block_manager.cpp:97-125); at least one token is always computed."""
    cache = CacheManager(NEEDS, 8, 16, 4, 256, prefix_cache=True)
    sched = Scheduler(SchedulerConfig(4, 64, 8, 16), cache)

    def step():
        plan = sched.schedule()
        for item in plan.sequences:
            s = item.sequence
            assert cache.computed(s.id) == item.token_start
            cache.reserve(s.id, item.token_start + item.token_count)
            cache.commit(s.id, item.token_start + item.token_count,
                         s.tokens[item.token_start:item.token_start + item.token_count])
        done = sched.postprocess(plan, [7 if i.samples else -1 for i in plan.sequences], lambda t: False)
        cache.audit()
        return plan, done

    sched.add(seq(1, 20, max_tokens=1))
    plan, done = step()
    assert shape(plan) == [(1, 0, 20, True)] and [d.id for d in done] == [1]
    sched.add(seq(2, 20, max_tokens=2))                  # same 20 tokens: two full pages are there
    sched.add(seq(3, 16, max_tokens=1))                  # ends on a page edge: its last page is computed
    plan, _ = step()
    assert shape(plan) == [(2, 16, 4, True), (3, 8, 8, True)]
    plan, done = step()
    assert shape(plan) == [(2, 20, 1, False)] and [d.id for d in done] == [2]
    assert cache.free_pages() == {None: 16} and cache.prefix_hit_pages == 3


def test_steps_launched_ahead_of_their_tokens():
    """advance() at the launch of a step, the next step planned and launched before the first
    one's tokens are known, resolve() in the order of the launches: lengths count the PENDING
    tokens (two per request for a while), a request at its max_tokens is out of the next plan,
    and one that ends on an end-of-sequence token drops the PENDING token of the step launched
    meanwhile, whose row has run for nothing."""
    from tiny_llm_infer_b200.engine.scheduler import PENDING
    sched, cache = make(pages=8, budget=32, page=8)
    a = Sequence(1, list(range(5)), SamplingParams(max_tokens=3, ignore_eos=True))
    b = Sequence(2, list(range(7)), SamplingParams(max_tokens=50))
    sched.add(a)
    sched.add(b)

    def launch(plan):
        for item in plan.sequences:
            cache.reserve(item.sequence.id, item.token_start + item.token_count)
            cache.commit(item.sequence.id, item.token_start + item.token_count)
        sched.advance(plan)

    first = sched.schedule()
    launch(first)
    assert a.tokens[-1] == PENDING and a.pending == 1 and len(a) == 6 and a.num_cached_tokens == 5
    second = sched.schedule()                        # made and launched while `first` runs
    assert shape(second) == [(1, 5, 1, False), (2, 7, 1, False)]
    launch(second)
    assert a.pending == 2 and a.tokens[-2:] == [PENDING, PENDING] and len(b) == 9
    assert sched.resolve(first, [11, 12], lambda t: t == 99) == []
    assert a.tokens[-2:] == [11, PENDING] and b.tokens[-2:] == [12, PENDING] and a.pending == 1
    third = sched.schedule()
    launch(third)                                    # a reaches max_tokens with it: over, pages back at once
    assert a.status is Status.FINISHED and not cache.has(1) and cache.has(2) and a.pending == 2
    done = sched.resolve(second, [13, 99], lambda t: t == 99)     # b ends here, with `third` under way
    assert [s.id for s in done] == [2] and b.completion == [12, 99] and b.pending == 0
    assert b.status is Status.FINISHED and not cache.has(2) and sched.is_finished()
    done = sched.resolve(third, [14, 5], lambda t: t == 99)       # b's row ran for nothing
    assert [s.id for s in done] == [1] and a.completion == [11, 13, 14] and b.completion == [12, 99]
    cache.audit()
    assert cache.free_pages() == {None: 8}


def test_a_plan_that_is_taken_back_leaves_the_queues_as_they_were():
    """``abort``: the step of a plan never ran.  Requests whose prompts it would have completed wait
    again (and are not decoded from a cache that lacks their prompt), the order of both queues is
    the old one, a request added meanwhile is kept, and the steps after it are those of a run in
    which the plan was never made."""
    def fresh():
        sched, cache = make(pages=32, budget=32)
        for i, n in enumerate((40, 9, 70)):
            sched.add(seq(i + 1, n))
        run_step(sched, cache)
        run_step(sched, cache)                       # 2 is running now, 1 and 3 are partly computed
        return sched, cache

    clean, clean_cache = fresh()
    want = [shape(run_step(clean, clean_cache)[0]) for _ in range(6)]

    sched, cache = fresh()
    running, waiting = list(sched.running), list(sched.waiting)
    plan = sched.schedule()                          # would complete request 1's prompt
    assert any(s.is_prefill and s.samples for s in plan.sequences)
    late = seq(9, 3)
    sched.add(late)
    sched.abort(plan)
    assert list(sched.running) == running and list(sched.waiting) == waiting + [late]
    assert all(s.status is Status.WAITING and s.num_scheduled_tokens == 0 for s in waiting)
    assert plan.sequences == []
    sched.waiting.remove(late)
    got = [shape(run_step(sched, cache)[0]) for _ in range(6)]
    assert got == want
    cache.audit()


def test_a_plan_that_fails_half_made_changes_nothing():
    """The second waiting prompt is larger than the pool: ``schedule`` raises, and the first, whose
    prompt the half-made plan had completed, is still waiting with nothing scheduled."""
    sched, cache = make(pages=4, page=8, budget=64)
    first, huge = seq(1, 9), seq(2, 40)
    sched.add(first)
    sched.add(huge)
    with pytest.raises(SchedulerError, match="needs 5 pages, the pool has 4"):
        sched.schedule()
    assert list(sched.waiting) == [first, huge] and not sched.running
    assert first.status is Status.WAITING and first.num_scheduled_tokens == 0
    sched.waiting.remove(huge)
    plan, _ = run_step(sched, cache)
    assert shape(plan) == [(1, 0, 9, True)]
