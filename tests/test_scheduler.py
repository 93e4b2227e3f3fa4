"""The scheduler's decisions, on the CPU, with a stand-in for the model: admission, portions under the token budget,
decoding, finishing, freeing, and what happens when pages run out."""

import random

import pytest

from oxr_inference_b200.cache import CacheManager, make_cache_plan
from oxr_inference_b200.engine.scheduler import Busy, Scheduler
from oxr_inference_b200.parts.base import PagedKVNeed
from oxr_inference_b200.sampling import SamplingParams

EOS = 99


def _scheduler(num_pages=64, page_size=4, max_running=4, max_step_tokens=32, prefill_chunk=16, max_positions=1000, max_waiting=100):
    plan = make_cache_plan([PagedKVNeed(1, 16, 0)], [None])
    cache = CacheManager(plan, page_size=page_size, num_pages=num_pages, max_requests=max_running)
    return Scheduler(cache, max_running=max_running, max_waiting=max_waiting, max_step_tokens=max_step_tokens,
                     prefill_chunk=prefill_chunk, max_positions=max_positions, eos_token_ids=(EOS,))


def _next_token(request):
    """Stand-in model: the next token is a function of everything so far, so a recomputed request must go on
    exactly as it would have."""
    return (sum(request.tokens) * 31 + len(request.tokens)) % 90


def _run(s, limit=10_000, on_step=None):
    done = []
    steps = 0
    while s.has_work():
        plan = s.schedule()
        done += plan.finished
        if on_step:
            on_step(plan)
        sampled = {p.request.id: _next_token(p.request) for p in plan.entries if p.wants_logits}
        done += s.commit(plan, sampled)
        s.cache.check()
        steps += 1
        assert steps < limit
    return done, steps


def _expected(prompt, n):
    class R:
        pass
    r = R()
    r.tokens = list(prompt)
    out = []
    for _ in range(n):
        t = (sum(r.tokens) * 31 + len(r.tokens)) % 90
        out.append(t)
        r.tokens.append(t)
    return out


def test_prompts_are_cut_under_the_budget_and_logits_wanted_only_at_the_end():
    s = _scheduler(max_step_tokens=20, prefill_chunk=16)
    a = s.add(list(range(40)), SamplingParams(max_tokens=3))
    b = s.add(list(range(5)), SamplingParams(max_tokens=3))
    p1 = s.schedule()
    assert [(p.request.id, p.start, p.count, p.wants_logits) for p in p1.entries] == [(0, 0, 16, False), (1, 0, 4, False)]
    s.commit(p1, {})
    p2 = s.schedule()
    # the running prompts go on in admission order; b's last token ends its prompt and wants logits
    assert [(p.request.id, p.start, p.count, p.wants_logits) for p in p2.entries] == [(0, 16, 16, False), (1, 4, 1, True)]
    s.commit(p2, {1: 7})
    p3 = s.schedule()
    # decodes first (b), then a's remaining portion
    assert [(p.request.id, p.start, p.count, p.wants_logits) for p in p3.entries] == [(0, 32, 8, True), (1, 5, 1, True)]
    assert not p3.decode_only
    s.commit(p3, {0: 1, 1: 2})
    p4 = s.schedule()
    assert p4.decode_only and p4.tokens == 2
    assert a.output == [1] and b.output == [7, 2]


def test_generation_is_what_the_model_gives_and_everything_is_freed():
    s = _scheduler()
    prompts = [[1, 2, 3], list(range(30)), [5], list(range(50, 77))]
    reqs = [s.add(p, SamplingParams(max_tokens=6)) for p in prompts]
    done, _ = _run(s)
    assert {r.id for r in done} == {0, 1, 2, 3}
    for r, p in zip(reqs, prompts):
        assert r.output == _expected(p, 6) and r.finish_reason == "length" and r.cache is None
    assert s.cache.free_pages == s.cache.usable_pages and s.cache.free_slots == 4


def test_eos_stops_and_is_not_kept_unless_ignored():
    s = _scheduler()
    r = s.add([1], SamplingParams(max_tokens=50))
    q = s.add([2], SamplingParams(max_tokens=4, ignore_eos=True))
    t = s.add([3], SamplingParams(max_tokens=50, stop_token_ids=(5,)))
    plan = s.schedule()
    assert {x.id for x in s.commit(plan, {r.id: EOS, q.id: EOS, t.id: 5})} == {r.id, t.id}
    assert r.output == [] and r.finish_reason == "stop" and t.finish_reason == "stop" and q.output == [EOS]


def test_position_limit_ends_a_request():
    s = _scheduler(max_positions=8)
    r = s.add([1, 2, 3, 4, 5], SamplingParams(max_tokens=50))
    _run(s)
    assert len(r.output) == 3 and r.finish_reason == "length"
    with pytest.raises(ValueError, match="position limit"):
        s.add(list(range(8)), SamplingParams())
    with pytest.raises(ValueError, match="at least one"):
        s.add([], SamplingParams())


def test_queue_limit_and_max_running():
    s = _scheduler(max_running=2, max_waiting=3)
    for i in range(3):
        s.add([i + 1], SamplingParams(max_tokens=2))
    with pytest.raises(Busy):
        s.add([9], SamplingParams())
    plan = s.schedule()
    assert len(plan.entries) == 2 and len(s.waiting) == 1, "head of the queue waits for a running slot"
    done, _ = _run(s)
    assert len(done) == 3


def test_admission_keeps_one_spare_page_per_running_request():
    # oxr_runtime/engine.py:438-441: a newcomer must leave a page of head-room for each request already running
    s = _scheduler(num_pages=7, page_size=4, max_step_tokens=64, prefill_chunk=64)  # 6 usable pages
    s.add(list(range(8)), SamplingParams(max_tokens=30))    # 2 pages
    s.add(list(range(12)), SamplingParams(max_tokens=30))   # 3 pages: 4 free - 3 = 1 >= 1 running -> admitted
    s.add(list(range(4)), SamplingParams(max_tokens=30))    # 1 page: 1 free - 1 = 0 < 2 running -> waits
    plan = s.schedule()
    assert [p.request.id for p in plan.entries] == [0, 1] and len(s.waiting) == 1


def test_pages_run_out_the_newest_request_is_preempted_and_recomputed_with_its_output_kept():
    s = _scheduler(num_pages=9, page_size=4, max_running=3, max_step_tokens=64, prefill_chunk=64)  # 8 usable pages = 32 tokens
    prompts = [list(range(10)), list(range(20, 29)), list(range(40, 47))]
    reqs = [s.add(p, SamplingParams(max_tokens=14)) for p in prompts]
    seen_preempted = []
    order = []  # admission order of the requests that hold pages

    def watch(plan):
        for victim in plan.preempted:
            seen_preempted.append(victim.id)
            assert victim.cache is None
            kept = [r.id for r in s.running if r.id in order]
            assert all(order.index(k) < order.index(victim.id) for k in kept), \
                "the victim is the most recently admitted running request (oxr_runtime/engine.py:610-627)"
            order.remove(victim.id)
        if plan.preempted:
            assert s.waiting and s.waiting[0].id in seen_preempted or any(p.request.id in seen_preempted and p.start == 0 for p in plan.entries), \
                "the victim goes to the front of the queue"
        for p in plan.entries:
            if p.start == 0 and p.request.id not in order:
                order.append(p.request.id)
    done, _ = _run(s, on_step=watch)
    assert s.preemptions > 0 and seen_preempted, "this workload cannot run without pushing a request out"
    for r, p in zip(reqs, prompts):
        assert r.output == _expected(p, 14), "a preempted request goes on exactly where it was"
        assert r.finish_reason == "length"
    assert any(r.preemptions for r in reqs)
    assert s.cache.free_pages == s.cache.usable_pages


def test_a_request_larger_than_the_whole_cache_ends_with_length():
    s = _scheduler(num_pages=4, page_size=4, max_running=2, max_step_tokens=64, prefill_chunk=64)  # 12 tokens of cache
    r = s.add(list(range(6)), SamplingParams(max_tokens=100))
    done, _ = _run(s)
    assert done == [r] and r.finish_reason == "length" and 1 <= len(r.output) <= 7
    assert r.output == _expected(list(range(6)), len(r.output))
    big = s.add(list(range(30)), SamplingParams(max_tokens=5))  # the prompt alone is beyond the cache
    done, _ = _run(s)
    assert done == [big] and big.finish_reason == "length" and big.output == []
    assert s.cache.free_pages == s.cache.usable_pages


def test_cancel_frees_pages():
    s = _scheduler()
    a = s.add(list(range(10)), SamplingParams(max_tokens=50))
    b = s.add(list(range(10)), SamplingParams(max_tokens=50))
    s.commit(s.schedule(), {a.id: 1, b.id: 2})
    a.cancel()
    plan = s.schedule()
    assert a in plan.finished and a.finish_reason == "cancelled" and a.cache is None
    assert [p.request.id for p in plan.entries] == [b.id]


def test_a_failed_step_fails_the_running_requests_and_frees_them():
    s = _scheduler()
    a = s.add([1, 2, 3], SamplingParams())
    s.schedule()
    failed = s.fail_running()
    assert failed == [a] and a.finish_reason == "error" and s.cache.free_pages == s.cache.usable_pages and not s.has_work()


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_under_page_pressure(seed):
    rng = random.Random(seed)
    s = _scheduler(num_pages=rng.choice([12, 20, 40]), page_size=rng.choice([2, 4, 8]), max_running=rng.choice([2, 3, 6]),
                   max_step_tokens=rng.choice([8, 24, 64]), prefill_chunk=rng.choice([3, 16, 64]))
    work = []
    for _ in range(25):
        prompt = [rng.randrange(90) for _ in range(rng.choice([1, 2, 5, 9, 17, 30]))]
        n = rng.choice([1, 3, 8, 20])
        work.append((s.add(prompt, SamplingParams(max_tokens=n)), prompt, n))
    _run(s)
    cap = s.cache.usable_pages * s.cache.page_size
    for r, prompt, n in work:
        if len(prompt) + n <= cap:
            assert r.finish_reason == "length" and r.output == _expected(prompt, n)
        else:
            assert r.output == _expected(prompt, len(r.output))
    assert s.cache.free_pages == s.cache.usable_pages and s.cache.free_slots == s.max_running


def test_tokens_from_equals_a_slice_of_the_joined_lists():
    from oxr_inference_b200.engine.scheduler import Request
    from oxr_inference_b200.sampling import SamplingParams

    r = Request(1, [10, 11, 12, 13], SamplingParams(), output=[20, 21, 22])
    for start in range(8):
        for count in range(0, 8 - start):
            assert r.tokens_from(start, count) == r.tokens[start:start + count]
    # two requests with equal fields are still two requests
    twin = Request(1, [10, 11, 12, 13], SamplingParams(), output=[20, 21, 22])
    assert r != twin and [r, twin].index(twin) == 1


def test_a_portion_that_does_not_finish_its_prompt_is_trimmed_to_whole_tile_rows():
    """32 running requests decode (32 tokens), a 4,096-token prompt gets portions: 2,048 would make the step 2,080 tokens,
    nine GEMM tile rows of 256; it gets 2,016 (eight rows), then 2,016 again, then its last 64."""
    from oxr_inference_b200.engine.scheduler import Scheduler

    s = Scheduler.__new__(Scheduler)
    s.prefill_chunk, s.max_step_tokens, s.step_tile = 2048, 2080, 256

    class R:
        def __init__(self, pending, skipped=0):
            self.pending, self.skipped = pending, skipped
    assert s._portion(R(4096), 2080 - 32) == 2016
    assert s._portion(R(2080), 2080 - 32) == 2016
    assert s._portion(R(64), 2080 - 32) == 64              # a portion that finishes the prompt is never trimmed
    assert s._portion(R(2048), 2080 - 32) == 2048
    assert s._portion(R(4096), 2080) == 2048               # nothing else in the step: already whole rows
    assert s._portion(R(4096), 300) == 300                 # small portions of a short step are left alone
    assert s._portion(R(4096), 32) == 0                    # but a sliver after 2,048 tokens would open a ninth tile row
    assert s._portion(R(20), 32) == 20                     # unless it finishes its prompt
    assert s._portion(R(4096, skipped=1), 32) == 32        # or it got nothing in the step before either
    s.prefill_chunk, s.max_step_tokens = 1000, 2048
    assert s._portion(R(4096), 2048 - 40) == 1000 - (40 + 1000) % 256   # 1040 -> 1024 tokens in the step
    s.step_tile = 0                                        # no tile size given: portions are what chunk and budget allow
    assert s._portion(R(4096), 2048 - 40) == 1000 and s._portion(R(4096), 8) == 8


def test_a_prompt_is_not_skipped_two_steps_in_a_row_by_the_sliver_rule():
    """Decoding requests nearly fill a long step; what is left is less than a tile row. The running prompt is passed
    over once, then takes its sliver."""
    plan = make_cache_plan([PagedKVNeed(1, 16, 0)], [None])
    cache = CacheManager(plan, page_size=4, num_pages=4000, max_requests=600)
    s = Scheduler(cache, max_running=600, max_waiting=1000, max_step_tokens=560, prefill_chunk=64, max_positions=10000,
                  eos_token_ids=(), step_tile=256)
    for _ in range(540):
        s.add([1], SamplingParams(max_tokens=50, ignore_eos=True))
    long_one = s.add(list(range(3, 80)) * 8, SamplingParams(max_tokens=2, ignore_eos=True))
    got = []
    for _ in range(8):
        plan_ = s.schedule()
        got.append(sum(p.count for p in plan_.entries if p.request is long_one))
        s.commit(plan_, {p.request.id: 5 for p in plan_.entries if p.wants_logits})
        s.cache.check()
    zeros = [i for i, c in enumerate(got) if c == 0]
    assert zeros and all(b - a > 1 for a, b in zip(zeros, zeros[1:])), f"portions per step: {got}"
    assert sum(got) > 0 and all(c in (0, 20) for c in got), f"portions per step: {got}"


def test_tokens_of_a_request_preempted_inside_a_step_go_back_into_the_budget():
    """A decoding request needs a page, the newest request (already chosen for this step) is preempted: its token is no
    longer counted against the step."""
    s = _scheduler(num_pages=5, page_size=4, max_running=3, max_step_tokens=3, prefill_chunk=16)
    a = s.add([1, 2, 3], SamplingParams(max_tokens=40, ignore_eos=True))
    b = s.add([4, 5, 6], SamplingParams(max_tokens=40, ignore_eos=True))
    # run until both decode and the pool (4 usable pages) is full
    for _ in range(200):
        plan_ = s.schedule()
        s.commit(plan_, {p.request.id: 7 for p in plan_.entries if p.wants_logits})
        s.cache.check()
        if plan_.preempted:
            break
    else:
        raise AssertionError("no preemption happened")
    assert plan_.preempted == [b] and [p.request for p in plan_.entries] == [a]
    assert sum(p.count for p in plan_.entries) == 1
