"""The scheduler's decisions, driven by a fake step function on the CPU: order within a step,
token budget, portions, admission, priority, finishing, and what happens when pages run out
(preemption by recomputation)."""
import pytest

from dispec_b200.cache import CacheGroupSpec, CacheManager
from dispec_b200.engine.scheduler import Scheduler, State
from dispec_b200.sampling import SamplingParams

VOCAB = 97


def make(pages=64, page_size=4, budget=2048, chunk=None, slots=16, groups=None):
    cache = CacheManager(groups or [CacheGroupSpec.key_value(1, 8)], page_size, pages, slots)
    return Scheduler(cache, max_batch_tokens=budget, chunk_size=chunk), cache


class FakeModel:
    """Next token = a hash of everything the request has stored so far: any token lost,
    repeated or fed at the wrong place changes the output."""

    def __init__(self):
        self.stored = {}

    def step(self, plan, cache):
        out = {}
        for e in plan.entries:
            seq = self.stored.setdefault(e.req_id, [])
            assert e.start == len(seq), "tokens fed at the wrong position"
            seq.extend(e.tokens)
            cache.commit(e.req_id, len(seq))
            if e.want:
                h = 7
                for i, t in enumerate(seq):
                    h = (h * 31 + t * (i + 1)) % 1000003
                out[e.req_id] = h % VOCAB
        return [out[r.id] for r in plan.sampled]

    def forget(self, req_id):
        self.stored.pop(req_id, None)


def run(sched, cache, model, max_steps=10000):
    steps = 0
    while sched.has_work() and steps < max_steps:
        plan = sched.schedule()
        cache.check()
        assert plan.entries, "a step with work scheduled nothing"
        tokens = model.step(plan, cache)
        for r in sched.process(plan, tokens):
            model.forget(r.id)
        steps += 1
    assert not sched.has_work()
    return steps


def wire(sched, cache, model):
    """Route frees through the fake model so that a preempted request starts over."""
    def on_free(rid):
        model.forget(rid)
        return cache.free(rid)
    sched._on_free = on_free


def expected(prompt, n, eos=None):
    m = FakeModel()
    seq = list(prompt)
    out = []
    while len(out) < n:
        h = 7
        for i, t in enumerate(seq):
            h = (h * 31 + t * (i + 1)) % 1000003
        out.append(h % VOCAB)
        seq.append(out[-1])
        if eos is not None and out[-1] == eos:
            break
    return out


def test_decodes_first_then_prompts_and_only_a_finished_prompt_yields_a_token():
    sched, cache = make(chunk=8)
    model = FakeModel()
    a = sched.add_request(list(range(5)), 4)
    plan = sched.schedule()
    assert [(e.req_id, len(e.tokens), e.want) for e in plan.entries] == [(a, 5, [4])]
    sched.process(plan, model.step(plan, cache))
    b = sched.add_request(list(range(20)), 3)
    plan = sched.schedule()  # a decodes, b's first portion of 8 yields nothing
    assert [(e.req_id, len(e.tokens), e.want) for e in plan.entries] == [(a, 1, [0]), (b, 8, [])]
    assert [r.id for r in plan.sampled] == [a]
    assert sched.prefilling[0].id == b and sched.prefilling[0].state == State.PREFILLING
    sched.process(plan, model.step(plan, cache))
    plan = sched.schedule()
    assert [(e.req_id, e.start, len(e.tokens)) for e in plan.entries] == [(a, 6, 1), (b, 8, 8)]
    sched.process(plan, model.step(plan, cache))
    plan = sched.schedule()  # last portion of b: 4 tokens, now it samples
    assert [(e.req_id, e.start, len(e.tokens), e.want) for e in plan.entries] == [(a, 7, 1, [0]), (b, 16, 4, [3])]
    assert [r.id for r in plan.sampled] == [a, b]
    sched.process(plan, model.step(plan, cache))
    assert sched.finished[0].id == a and sched.finished[0].output_ids == expected(range(5), 4)
    run(sched, cache, model)
    assert sched.collect_outputs()[b] == expected(range(20), 3)
    assert sched.num_prefill_tokens == 25 and sched.num_decode_tokens == 3 + 2
    assert cache.num_free_pages() == 64


def test_token_budget_bounds_a_step_and_skipped_decodes_catch_up():
    sched, cache = make(budget=2)
    model = FakeModel()
    wire(sched, cache, model)
    ids = [sched.add_request([i, i + 1], 5) for i in range(3)]
    seen = []
    while sched.has_work():
        plan = sched.schedule()
        seen.append(sum(len(e.tokens) for e in plan.entries))
        sched.process(plan, model.step(plan, cache))
    assert max(seen) <= 2
    for i, rid in enumerate(ids):
        assert sched.collect_outputs()[rid] == expected([i, i + 1], 5)


def test_priority_then_age_and_head_of_line_admission():
    sched, cache = make(pages=6, page_size=4, slots=8)  # 24 tokens of cache
    model = FakeModel()
    wire(sched, cache, model)
    low = sched.add_request(list(range(14)), 2, priority=0)  # 4 pages, room for its 2 tokens
    high = sched.add_request(list(range(6)), 2, priority=5)  # 2 pages, room for its 2 tokens
    tail = sched.add_request([1], 2, priority=0)  # would fit, but waits behind `low`
    plan = sched.schedule()
    assert [e.req_id for e in plan.entries] == [high, low]
    sched.process(plan, model.step(plan, cache))
    late = sched.add_request(list(range(12)), 2, priority=9)  # 3 pages: does not fit yet
    plan = sched.schedule()
    assert sorted(e.req_id for e in plan.entries) == [low, high]  # `late` blocks `tail` too
    assert [r.id for r in sched.waiting] == [late, tail]
    sched.process(plan, model.step(plan, cache))
    run(sched, cache, model)
    assert sched.collect_outputs()[tail] == expected([1], 2)
    assert sched.collect_outputs()[late] == expected(range(12), 2)


def test_end_of_sequence_token_is_kept_and_stops_the_request():
    sched, cache = make()
    model = FakeModel()
    want = expected([3, 4, 5], 50)
    eos = want[6]
    first = want.index(eos)
    rid = sched.add_request([3, 4, 5], 50, eos_id=eos)
    run(sched, cache, model)
    out = sched.collect_outputs()[rid]
    assert out == want[:first + 1] and sched.finished[0].finish_reason == "stop"


def test_running_out_of_pages_preempts_the_newest_and_recomputes():
    # 3 pages of 16 tokens, two 16-token prompts, 24 new tokens each: the reference raises out
    # of step() here (dispec/sched/scheduler.py:137 lets OutOfBlocksError through)
    sched, cache = make(pages=3, page_size=16)
    model = FakeModel()
    wire(sched, cache, model)
    a = sched.add_request(list(range(16)), 24)
    b = sched.add_request(list(range(100, 116)), 24)
    steps = run(sched, cache, model)
    out = sched.collect_outputs()
    assert out[a] == expected(range(16), 24)
    assert out[b] == expected(range(100, 116), 24)
    assert sched.num_preemptions >= 1 and steps < 200
    by_id = {r.id: r for r in sched.finished}
    assert by_id[b].num_preemptions >= 1 and by_id[a].num_preemptions == 0  # the older one goes on
    cache.check()
    assert cache.num_free_pages() == 3 and cache.free_slots() == 16


def test_many_requests_through_a_small_pool_all_finish_with_the_right_tokens():
    sched, cache = make(pages=10, page_size=4, budget=24, chunk=8, slots=6)
    model = FakeModel()
    wire(sched, cache, model)
    specs = [([i * 3 + j for j in range(1 + (i * 7) % 19)], 3 + (i * 5) % 11) for i in range(14)]
    ids = [sched.add_request(p, n, SamplingParams()) for p, n in specs]
    run(sched, cache, model)
    out = sched.collect_outputs()
    for rid, (p, n) in zip(ids, specs):
        assert out[rid] == expected(p, n), rid
    cache.check()
    assert cache.num_free_pages() == 10


def test_window_group_requests_finish_under_their_promise():
    groups = [CacheGroupSpec.key_value(1, 8), CacheGroupSpec.key_value(1, 8, window=6)]
    sched, cache = make(pages=[40, 8], page_size=4, budget=16, chunk=8, slots=4, groups=groups)
    model = FakeModel()
    wire(sched, cache, model)
    ids = [sched.add_request(list(range(i, i + 30)), 20) for i in range(3)]
    run(sched, cache, model)
    for i, rid in enumerate(ids):
        assert sched.collect_outputs()[rid] == expected(range(i, i + 30), 20)
    assert cache.num_free_pages(1) == 8 and cache.pools[1].reserved == 0


def test_a_request_that_can_never_fit_is_refused():
    sched, _ = make(pages=2, page_size=4)
    with pytest.raises(ValueError, match="never fit"):
        sched.add_request(list(range(8)), 2)
    sched.add_request(list(range(8)), 1)  # 8 stored positions fit exactly
    with pytest.raises(ValueError):
        sched.add_request([], 2)


def test_window_pool_bounds_the_portions_and_a_pool_below_the_window_refuses():
    """Admission asks a window group for the most pages the request ever holds at once, which
    grows with the portion a step brings.  Portions are therefore capped by what the window
    group's pool holds beside the window, so that no request waits forever at the head of the
    queue (and blocks everything behind it); a pool that cannot even hold the window and one
    token refuses every request when it is added."""
    groups = [CacheGroupSpec.key_value(1, 8), CacheGroupSpec.key_value(1, 8, window=5)]
    sched, cache = make(pages=[20, 6], page_size=4, budget=32, slots=4, groups=groups)
    # window 5, six pages of 4: a portion of up to (6 - 1) * 4 - 5 + 1 = 16 tokens, not the budget's 32
    assert sched.max_portion == 16
    model = FakeModel()
    wire(sched, cache, model)
    a = sched.add_request(list(range(24)), 9)
    b = sched.add_request(list(range(10)), 15)
    plan = sched.schedule()
    assert [len(e.tokens) for e in plan.entries] == [16]  # and the window pool is promised to a alone
    for r in sched.process(plan, model.step(plan, cache)):
        model.forget(r.id)
    run(sched, cache, model)
    assert sched.collect_outputs()[a] == expected(range(24), 9)
    assert sched.collect_outputs()[b] == expected(range(10), 15)
    cache.check()
    tiny, _ = make(pages=[20, 2], page_size=4, budget=32, slots=4, groups=groups)
    with pytest.raises(ValueError, match="too small"):
        tiny.add_request([1, 2, 3], 2)


@pytest.mark.parametrize("seed", range(12))
def test_random_workloads_with_a_window_group_finish_or_are_refused(seed):
    """Random pools, windows, budgets and requests over a full and a window group: every request
    is either refused when added or finishes with the right tokens; no step with work left
    schedules nothing; every page and promise comes back."""
    import random
    rng = random.Random(1000 + seed)
    page_size = rng.choice([2, 4, 8])
    window = rng.choice([3, 5, 9, 17, 40])
    pages = [rng.randint(4, 24), rng.randint(3, 12)]
    groups = [CacheGroupSpec.key_value(1, 8), CacheGroupSpec.key_value(1, 8, window=window)]
    budget = rng.choice([4, 16, 32, 64])
    chunk = rng.choice([None, 3, 8, 20])
    sched, cache = make(pages=pages, page_size=page_size, budget=budget, chunk=chunk, slots=4, groups=groups)
    model = FakeModel()
    wire(sched, cache, model)
    accepted = {}
    for _ in range(rng.randint(3, 10)):
        prompt = [rng.randrange(VOCAB) for _ in range(rng.randint(1, 40))]
        new = rng.randint(1, 30)
        try:
            accepted[sched.add_request(prompt, new, priority=rng.choice([0, 0, 1]))] = (prompt, new)
        except ValueError:
            pass
    run(sched, cache, model)
    out = sched.collect_outputs()
    for rid, (prompt, new) in accepted.items():
        assert out[rid] == expected(prompt, new), rid
    cache.check()
    for g, pool in enumerate(cache.pools):
        assert pool.num_free == pool.num_pages and pool.reserved == 0, g


# ------------------------------------------------------------------- overlapped steps
def run_overlapped(sched, cache, model, max_steps=10000):
    """The engine's loop with one step in flight: step n + 1 is scheduled and run before the
    tokens of step n are resolved; an entry with feed_row takes its token from the result of
    the step before, as the device does."""
    inflight = None
    steps = 0
    wasted = 0

    def resolve(launched):
        for r in sched.resolve(*launched):
            model.forget(r.id)

    while (sched.has_work() or inflight) and steps < max_steps:
        if inflight and sched.needs_resolved_tokens():
            resolve(inflight)
            inflight = None
        plan = sched.schedule()
        cache.check()
        if not plan.entries:
            assert inflight, "a step with work scheduled nothing"
            resolve(inflight)
            inflight = None
            continue
        for e in plan.entries:
            if e.feed_row >= 0:
                assert e.tokens == [0] and inflight is not None
                e.tokens = [inflight[1][e.feed_row]]
        tokens = model.step(plan, cache)
        wasted += sum(1 for r in plan.sampled if r.state == State.FINISHED and r.finish_reason == "stop")
        sched.launched(plan)
        previous, inflight = inflight, (plan, tokens)
        if previous:
            resolve(previous)
        steps += 1
    assert not sched.has_work() and inflight is None
    return steps


def test_overlap_feeds_the_token_in_flight_by_its_row():
    from dispec_b200.engine.scheduler import PENDING
    sched, cache = make()
    a = sched.add_request([1, 2, 3], 4)
    b = sched.add_request([4, 5], 4)
    plan0 = sched.schedule()
    for e in plan0.entries:
        cache.commit(e.req_id, e.start + len(e.tokens))
    sched.launched(plan0)
    assert [r.output_ids for r in plan0.sampled] == [[PENDING], [PENDING]]
    plan1 = sched.schedule()
    assert [(e.req_id, e.tokens, e.feed_row) for e in plan1.entries] == [(a, [0], 0), (b, [0], 1)]
    for e in plan1.entries:
        cache.commit(e.req_id, e.start + 1)
    sched.launched(plan1)
    sched.resolve(plan0, [11, 12])
    assert [r.output_ids for r in plan0.sampled] == [[11, PENDING], [12, PENDING]]
    # the newest token is still in flight: fed again, from the rows of plan1
    plan2 = sched.schedule()
    assert [(e.tokens, e.feed_row) for e in plan2.entries] == [([0], 0), ([0], 1)]
    for e in plan2.entries:
        cache.commit(e.req_id, e.start + 1)
    sched.launched(plan2)
    sched.resolve(plan1, [21, 22])
    sched.resolve(plan2, [31, 32])
    plan3 = sched.schedule()  # everything resolved: tokens come from the host again
    assert [(e.tokens, e.feed_row) for e in plan3.entries] == [([31], -1), ([32], -1)]


def test_overlap_end_of_sequence_is_seen_one_step_late_and_length_at_once():
    sched, cache = make()
    model = FakeModel()
    wire(sched, cache, model)
    prompt = [5, 6, 7]
    full = expected(prompt, 12)
    eos = full[4]
    assert eos not in full[:4]
    stops = sched.add_request(prompt, 12, eos_id=eos)
    short = sched.add_request([9, 8], 3)
    free0 = cache.num_free_pages()
    steps = run_overlapped(sched, cache, model)
    out = sched.collect_outputs()
    assert out[stops] == full[:5] and out[short] == expected([9, 8], 3)
    by_id = {r.id: r for r in sched.finished}
    assert by_id[stops].finish_reason == "stop" and by_id[short].finish_reason == "length"
    # the request that stopped ran one step past its last token; nothing else did
    assert steps == 6
    assert cache.num_free_pages() == free0
    cache.check()


@pytest.mark.parametrize("seed", range(6))
def test_overlap_gives_the_same_tokens_as_waiting_for_every_step(seed):
    import random
    rnd = random.Random(seed)
    reqs = []
    for _ in range(12):
        prompt = [rnd.randrange(VOCAB) for _ in range(rnd.randrange(1, 30))]
        n = rnd.randrange(1, 20)
        eos = rnd.choice([None, None, rnd.randrange(VOCAB)])
        reqs.append((prompt, n, eos))
    outs = []
    for overlapped in (False, True):
        sched, cache = make(pages=40, page_size=4, budget=24, chunk=8)
        model = FakeModel()
        wire(sched, cache, model)
        ids = [sched.add_request(p, n, eos_id=e) for p, n, e in reqs]
        (run_overlapped if overlapped else run)(sched, cache, model)
        out = sched.collect_outputs()
        outs.append([out[i] for i in ids])
        assert cache.num_free_pages() == 40
        cache.check()
    assert outs[0] == outs[1]
    for (p, n, e), got in zip(reqs, outs[1]):
        assert got == expected(p, n, e)


def test_overlap_resolves_first_when_pages_are_short_and_never_preempts_a_pending_token():
    sched, cache = make(pages=6, page_size=4, budget=64)
    a = sched.add_request([1] * 8, 12)
    b = sched.add_request([2] * 8, 12)
    model = FakeModel()
    wire(sched, cache, model)
    plan = sched.schedule()
    model.step(plan, cache)
    sched.launched(plan)
    # 2 full pages each, 2 free, 2 running: enough for one more token each
    assert not sched.needs_resolved_tokens()
    plan2 = sched.schedule()
    tokens2 = None
    for e in plan2.entries:
        e.tokens = [3]
    tokens2 = model.step(plan2, cache)
    sched.launched(plan2)
    assert cache.min_free_pages() < 2 and sched.needs_resolved_tokens()
    with pytest.raises(RuntimeError):
        sched._preempt(sched.running[0])
    assert a != b and tokens2 is not None
