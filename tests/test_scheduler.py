"""Scheduler decisions on the CPU: admission, portions under a token budget,
mixed steps, finishing and freeing, and what happens when pages run out."""

import random

import pytest

from freetoken_b200.cache import CacheManager, PagedKVNeed
from freetoken_b200.engine.scheduler import Request, Scheduler
from freetoken_b200.sampling import SamplingParams


def make(num_pages=16, page=4, slots=4, max_seq_len=64, budget=8, eos=()):
    cache = CacheManager([PagedKVNeed(2, 16, None)], page, num_pages, slots, max_seq_len)
    return Scheduler(cache, budget, eos), cache


def run_step(sched, cache, token_of=lambda r: 7):
    """What the engine does with a plan: pages, advance, one token per sampling entry."""
    plan = sched.plan()
    for e in plan:
        cache.grow(e.request.id, cache.length(e.request.id) + len(e.tokens))
    for e in plan:
        cache.advance(e.request.id, len(e.tokens))
    done = sched.complete(plan, [token_of(e.request) for e in plan if e.samples])
    sched.check_integrity()
    return plan, done


def req(rid, n, max_tokens=4, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, **kw))


def test_prompt_is_cut_into_portions_under_the_token_budget():
    sched, cache = make(budget=8)
    sched.submit(req("a", 19, max_tokens=2))
    sizes, samples = [], []
    while sched.has_work():
        plan, _ = run_step(sched, cache)
        sizes.append([len(e.tokens) for e in plan])
        samples.append([e.samples for e in plan])
    assert sizes == [[8], [8], [3], [1]]                     # 19 = 8 + 8 + 3, then one decode step
    assert samples == [[False], [False], [True], [True]]
    r = sched.finished[0]
    assert r.output == [7, 7] and r.finish_reason == "length"
    assert cache.free_pages() == cache.total_pages() and cache.free_slots == 4


def test_decode_tokens_ride_beside_prompt_portions():
    sched, cache = make(budget=8)
    sched.submit(req("a", 3, max_tokens=6))
    run_step(sched, cache)                                    # a: whole prompt, first token
    sched.submit(req("b", 12, max_tokens=2))
    plan, _ = run_step(sched, cache)
    assert [(e.request.id, len(e.tokens), e.samples) for e in plan] == [("a", 1, True), ("b", 7, False)]
    plan, _ = run_step(sched, cache)                          # budget 8 = 1 decode + 5 left of b's prompt
    assert [(e.request.id, len(e.tokens), e.samples) for e in plan] == [("a", 1, True), ("b", 5, True)]
    plan, _ = run_step(sched, cache)
    assert sorted((e.request.id, len(e.tokens)) for e in plan) == [("a", 1), ("b", 1)]


def test_several_short_prompts_share_one_step_in_arrival_order():
    sched, cache = make(budget=10)
    for rid, n in (("a", 3), ("b", 4), ("c", 6)):
        sched.submit(req(rid, n))
    plan, _ = run_step(sched, cache)
    assert [(e.request.id, len(e.tokens), e.samples) for e in plan] == \
        [("a", 3, True), ("b", 4, True), ("c", 3, False)]


def test_when_pages_run_out_new_requests_wait_and_running_ones_never_starve():
    # 6 pages of 4 tokens; each request needs ceil((5 + 6) / 4) = 3 pages at worst
    sched, cache = make(num_pages=6, page=4, slots=4, budget=16)
    for rid in "abc":
        sched.submit(req(rid, 5, max_tokens=6))
    plan, _ = run_step(sched, cache)
    assert [e.request.id for e in plan] == ["a", "b"]        # c does not fit beside a's and b's worst case
    assert [r.id for r in sched.pending] == ["c"]
    steps = 0
    while sched.has_work():
        plan, done = run_step(sched, cache)
        steps += 1
        assert steps < 50
        if any(e.request.id == "c" for e in plan):
            assert {r.id for r in sched.finished} >= {"a"} or {r.id for r in sched.finished} >= {"b"}
    assert sorted(r.id for r in sched.finished) == ["a", "b", "c"]
    assert all(len(r.output) == 6 for r in sched.finished)
    assert cache.free_pages() == cache.total_pages()


def test_requests_that_can_never_run_are_refused_at_submit():
    sched, cache = make(num_pages=4, page=4, max_seq_len=40)
    too_long = req("long", 40)
    assert not sched.submit(too_long) and "max_seq_len" in too_long.finish_reason
    too_big = req("big", 10, max_tokens=20)                   # 30 tokens = 8 pages > 4
    assert not sched.submit(too_big) and "pages" in too_big.finish_reason
    empty = Request("e", [], SamplingParams())
    assert not sched.submit(empty)
    clamp = req("clamp", 10, max_tokens=1000)                 # room left: 40 - 10 = 30 -> 10 pages > 4
    assert not sched.submit(clamp)
    sched2, _ = make(num_pages=16, page=4, max_seq_len=40)
    ok = req("ok", 10, max_tokens=1000)
    assert sched2.submit(ok) and ok.max_tokens == 30          # clamped to the room left
    assert not sched.has_work()


def test_eos_stops_and_wins_over_length_unless_ignored():
    sched, cache = make(eos=[99])
    a, b, c = req("a", 2, max_tokens=3), req("b", 2, max_tokens=3, ignore_eos=True), req("c", 2, max_tokens=1)
    for r in (a, b, c):
        sched.submit(r)
    while sched.has_work():
        run_step(sched, cache, token_of=lambda r: 99)
    assert (a.output, a.finish_reason) == ([99], "stop")
    assert (b.output, b.finish_reason) == ([99, 99, 99], "length")
    assert (c.output, c.finish_reason) == ([99], "stop")      # EOS on the last allowed token: stop
    d = req("d", 2, max_tokens=5, stop_token_ids=[5])
    sched.submit(d)
    while sched.has_work():
        run_step(sched, cache, token_of=lambda r: 5)
    assert d.finish_reason == "stop"


def test_abort_gives_everything_back():
    sched, cache = make(budget=4)
    sched.submit(req("a", 10))
    sched.submit(req("b", 3))
    run_step(sched, cache)                                    # a is half-way through its prompt
    assert sched.abort("a") and sched.abort("b") and not sched.abort("nobody")
    sched.check_integrity()
    assert cache.free_pages() == cache.total_pages() and not sched.has_work()


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_with_nothing_left_behind(seed):
    rng = random.Random(seed)
    sched, cache = make(num_pages=rng.randint(8, 20), page=rng.choice([2, 4, 8]),
                        slots=rng.randint(1, 4), max_seq_len=64, budget=rng.randint(2, 12))
    accepted = []
    for i in range(12):
        r = req(f"r{i}", rng.randint(1, 30), max_tokens=rng.randint(1, 12))
        if sched.submit(r):
            accepted.append(r)
    steps = 0
    while sched.has_work():
        plan, _ = run_step(sched, cache, token_of=lambda r: rng.randint(0, 50))
        assert plan and sum(len(e.tokens) for e in plan if not e.samples or len(e.tokens) > 1) <= sched.max_step_tokens
        steps += 1
        assert steps < 2000
    assert all(r.finish_reason == "length" and len(r.output) == r.max_tokens for r in accepted)
    assert cache.free_pages() == cache.total_pages() and cache.free_slots == cache.max_slots


def _grow(cache, plan):
    for e in plan:
        cache.grow(e.request.id, cache.length(e.request.id) + len(e.tokens))
        cache.advance(e.request.id, len(e.tokens))


def test_a_step_planned_before_the_last_one_is_recorded_takes_its_token_from_the_device():
    sched, cache = make(budget=8)
    sched.submit(req("a", 3, max_tokens=3))
    p1 = sched.plan()                                 # whole prompt, first token in flight
    _grow(cache, p1)
    assert [(e.samples, e.from_device) for e in p1] == [(True, False)]
    p2 = sched.plan()                                 # planned ahead: input is the token on the device
    _grow(cache, p2)
    assert [(len(e.tokens), e.samples, e.from_device) for e in p2] == [(1, True, True)]
    assert sched.complete(p1, [11]) == []
    p3 = sched.plan()                                 # token 2 still in flight
    _grow(cache, p3)
    assert [e.from_device for e in p3] == [True]
    assert sched.plan() == []                         # three tokens planned: max_tokens reached
    assert sched.complete(p2, [12]) == []
    done = sched.complete(p3, [13])
    assert [r.id for r in done] == ["a"] and done[0].output == [11, 12, 13]
    assert done[0].finish_reason == "length" and done[0].inflight == 0
    sched.check_integrity()
    assert cache.free_pages() == cache.total_pages()


def test_a_token_computed_past_an_eos_is_dropped():
    sched, cache = make(budget=8, eos=[99])
    sched.submit(req("a", 2, max_tokens=6))
    sched.submit(req("b", 2, max_tokens=6))
    p1 = sched.plan()
    _grow(cache, p1)
    p2 = sched.plan()                                 # both planned ahead
    _grow(cache, p2)
    done = sched.complete(p1, [99, 5])                # a stopped; its entry in p2 is already running
    assert [r.id for r in done] == ["a"] and done[0].finish_reason == "stop"
    assert not cache.has_request("a")                 # what it held is given back at once
    p3 = sched.plan()
    _grow(cache, p3)
    assert [e.request.id for e in p3] == ["b"]
    assert sched.complete(p2, [42, 6]) == []          # a's extra token is dropped
    assert done[0].output == [99]
    assert sched.running[0].output == [5, 6]
    sched.check_integrity()


def test_a_stop_string_in_the_newest_text_stops_the_request():
    words = {1: "a", 2: "b", 3: " EN", 4: "D ", 5: "c"}
    cache = CacheManager([PagedKVNeed(2, 16, None)], 4, 16, 4, 64)
    sched = Scheduler(cache, 8, (), detokenize=lambda ids: "".join(words[i] for i in ids))
    sched.submit(Request("a", [1, 2], SamplingParams(max_tokens=10, stop_strs=["END", ""])))
    out = iter([1, 3, 4, 5, 5])
    while sched.has_work():
        run_step(sched, cache, token_of=lambda r: next(out))
    r = sched.finished[0]
    assert r.output == [1, 3, 4] and r.finish_reason == "stop"     # "a EN" + "D " holds "END"


@pytest.mark.parametrize("seed", range(6))
def test_planning_one_step_ahead_gives_the_same_outputs_as_the_synchronous_loop(seed):
    """A stand-in model whose next token is a function of the request and of how
    many tokens it has: the loop that plans step N+1 before it records step N
    must end with the same outputs, finish reasons and an empty cache as the loop
    that records each step at once - with stops that are only seen one step late."""
    def workload():
        rng = random.Random(seed)
        sched, cache = make(num_pages=rng.randint(10, 24), page=rng.choice([2, 4, 8]),
                            slots=rng.randint(1, 4), max_seq_len=64, budget=rng.randint(2, 12), eos=[0])
        reqs = [req(f"r{i}", rng.randint(1, 30), max_tokens=rng.randint(1, 12), ignore_eos=rng.random() < 0.3)
                for i in range(10)]
        return sched, cache, reqs

    def token_of(r, n_out):
        return (hash((r.id, n_out, seed)) % 7)          # 0 is the EOS: about one token in seven stops

    def run(ahead: bool):
        sched, cache, reqs = workload()
        for r in reqs:
            sched.submit(r)
        inflight = None                                   # (plan, tokens) of the step not yet recorded
        steps = 0
        while sched.has_work() or inflight is not None:
            steps += 1
            assert steps < 2000
            if not ahead and inflight is not None:
                sched.complete(*inflight)
                inflight = None
            plan = sched.plan()
            for e in plan:
                cache.grow(e.request.id, cache.length(e.request.id) + len(e.tokens))
                cache.advance(e.request.id, len(e.tokens))
            # the token a sampling entry yields: by how many tokens the request will have then
            tokens = [token_of(e.request, len(e.request.output) + e.request.inflight - 1) for e in plan if e.samples]
            if inflight is not None:
                sched.complete(*inflight)
            inflight = (plan, tokens) if plan else None
            sched.check_integrity()
        assert cache.free_pages() == cache.total_pages()
        return {r.id: (tuple(r.output), r.finish_reason) for r in reqs}

    assert run(ahead=True) == run(ahead=False)


def test_status_lines_follow_the_reference_wording():
    """One line per step with prompt tokens, one per N decode-only steps."""
    from freetoken_b200.engine.scheduler import PlannedEntry
    from freetoken_b200.engine.status import StatusReporter
    lines, now = [], [0.0]
    rep = StatusReporter(lines.append, clock=lambda: now[0], decode_log_interval=3)
    r = Request("a", [1, 2, 3], SamplingParams(max_tokens=4))
    now[0] = 0.5
    rep.report([PlannedEntry(r, [1, 2, 3], True)], running=0, queued=2, pages_used=1, pages_total=4, page_size=16)
    assert lines == ["Prefill batch, #new-seq: 1, #new-token: 3, #cached-token: 0, token usage: 0.25, "
                     "#running-req: 0, #queue-req: 2, input throughput (token/s): 6.00"]
    for step in range(3):
        now[0] += 1.0
        rep.report([PlannedEntry(r, [7], True)], running=1, queued=0, pages_used=2, pages_total=4, page_size=16)
    assert len(lines) == 2
    # 1 token sampled by the prompt's last portion + 3 decoded, over the 3.5 s since the reporter began
    assert lines[1] == ("Decode batch, #running-req: 1, #token: 32, token usage: 0.50, "
                        "gen throughput (token/s): 1.14, #queue-req: 0")
