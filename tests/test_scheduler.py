"""The scheduler's decisions (host code, no GPU): a fake model picks the tokens."""

from __future__ import annotations

import pytest

from llm_inference_b200.csrc.host_module import host


def make(h, *, pages=16, page=4, seqs=3, context=64, budget=12, chunk=4, burst=8, vocab=50):
    cache = h.CacheManager(page, [h.GroupSpec("full", pages, 0)], 0, burst)
    return cache, h.Scheduler(cache, seqs, context, budget, chunk, burst, vocab, 1)


def run_step(s, pick=lambda entry: 9):
    plan = s.plan()
    tokens = [pick(e) for e in plan.entries if e.wants_token]
    return plan, s.commit(plan, tokens)


def test_lifecycle_portions_and_first_token():
    h = host()
    cache, s = make(h)
    rid = s.submit(list(range(11)), 3, [], h.SamplingParams())
    assert s.request(rid).state == "waiting"
    plan, events = run_step(s)
    # Nothing decodes, so the portion is the burst size (8); the prompt is not done yet.
    assert [(e.start, e.count, e.wants_token, e.decode) for e in plan.entries] == [(0, 8, False, False)]
    assert events == [] and s.request(rid).state == "prefilling"
    plan, events = run_step(s)
    assert [(e.start, e.count, e.wants_token) for e in plan.entries] == [(8, 3, True)]
    assert plan.tokens.tolist() == [8, 9, 10]
    assert [(e.token, e.finished) for e in events] == [(9, False)] and s.request(rid).state == "running"
    plan, events = run_step(s, lambda e: 7)
    assert [(e.start, e.count, e.decode) for e in plan.entries] == [(11, 1, True)] and plan.tokens.tolist() == [9]
    plan, events = run_step(s, lambda e: 8)
    assert events[0].finished and events[0].reason == "length"
    request = s.request(rid)
    assert request.state == "completed" and request.output == [9, 7, 8]
    assert cache.stats()["kv_pools"]["full"]["used_pages"] == 0 and not s.has_work()
    s.forget(rid)
    with pytest.raises(IndexError):
        s.request(rid)


def test_decode_first_then_prompt_portions_under_the_budget():
    h = host()
    cache, s = make(h, budget=7, chunk=4, burst=6)
    a = s.submit([1] * 6, 5, [], h.SamplingParams())
    run_step(s)  # a: whole prompt in one burst, first token
    b = s.submit([2] * 9, 2, [], h.SamplingParams())
    c = s.submit([3] * 5, 2, [], h.SamplingParams())
    plan, _ = run_step(s)
    # One decode token, then b's chunk (4), then what is left of the budget (2) for c.
    assert [(e.request_id, e.count, e.decode) for e in plan.entries] == [(a, 1, True), (b, 4, False), (c, 2, False)]
    assert plan.total_tokens == 7
    plan, _ = run_step(s)
    assert [(e.request_id, e.start, e.count) for e in plan.entries] == [(a, 7, 1), (b, 4, 4), (c, 2, 2)]
    plan, events = run_step(s)
    assert [(e.request_id, e.start, e.count, e.wants_token) for e in plan.entries] == [
        (a, 8, 1, True), (b, 8, 1, True), (c, 4, 1, True)]
    assert sorted(e.request_id for e in events) == [a, b, c]


def test_stop_token_context_limit_and_forced_tokens():
    h = host()
    cache, s = make(h, context=8)
    a = s.submit([1, 2, 3], 5, [4], h.SamplingParams())
    _, events = run_step(s, lambda e: 4)
    assert events[0].reason == "stop" and s.request(a).output == [4]
    b = s.submit([1, 2, 3, 4, 5], 3, [], h.SamplingParams())
    run_step(s)
    _, events = run_step(s)
    _, events = run_step(s)
    # length 7 after the third token's step: 7 + 1 >= 8
    assert events[0].finished and events[0].reason in ("context", "length")
    c = s.submit([1, 2, 3, 4, 5, 6], 2, [], h.SamplingParams())
    run_step(s)
    _, events = run_step(s)
    assert events[0].reason == "length" or events[0].reason == "context"
    d = s.submit([1], 3, [], h.SamplingParams())
    s.force(d, [30, 31])
    outputs = []
    while s.has_work():
        _, events = run_step(s, lambda e: 9)
        outputs += [e.token for e in events]
    assert outputs == [30, 31, 9]


def test_budget_that_ends_at_the_context_limit():
    h = host()
    cache, s = make(h, context=6)
    with pytest.raises(ValueError, match="exceed the 6-token context"):
        s.submit([1, 2, 3], 4, [], h.SamplingParams())
    s.submit([1, 2, 3], 3, [], h.SamplingParams())
    reasons = []
    while s.has_work():
        _, events = run_step(s)
        reasons += [e.reason for e in events]
    # The token budget and the context end together; the budget is reported first, as in
    # the reference's order of checks (python/instinct/mlx_engine.py:517-524).
    assert reasons == ["", "", "length"]


def test_invalid_requests_are_refused_at_submit():
    h = host()
    cache, s = make(h, pages=4, context=64)
    p = h.SamplingParams()
    for prompt, new, stop, message in [
        ([], 1, [], "non-empty"),
        ([50], 1, [], "outside the vocabulary"),
        ([-1], 1, [], "outside the vocabulary"),
        ([1], 1, [99], "outside the vocabulary"),
        ([1], 0, [], "positive integer"),
        ([1] * 60, 5, [], "exceed the 64-token context"),
        ([1] * 10, 7, [], "more K/V memory than the cache has"),  # 17 tokens = 5 pages > 4
    ]:
        with pytest.raises(ValueError, match=message):
            s.submit(prompt, new, stop, p)
    assert s.stats()["submitted"] == 0 and s.stats()["rejected"] == 1
    for bad in [dict(temperature=-1.0), dict(temperature=11.0), dict(top_p=0.0), dict(top_p=1.5), dict(top_k=-1), dict(min_p=1.0)]:
        with pytest.raises(ValueError):
            h.SamplingParams(**bad)


def test_when_pages_run_out_requests_wait_in_order():
    h = host()
    cache, s = make(h, pages=6, page=4, seqs=4, budget=32, chunk=8, burst=8)
    p = h.SamplingParams()
    a = s.submit([1] * 8, 8, [], p)  # 4 pages
    b = s.submit([2] * 8, 4, [], p)  # 3 pages: does not fit beside a
    c = s.submit([3] * 2, 2, [], p)  # 1 page: would fit, but may not overtake b
    plan, _ = run_step(s)
    assert [e.request_id for e in plan.entries] == [a]
    assert s.request(b).state == "waiting" and s.request(c).state == "waiting"
    assert cache.stats()["allocation_failures"] >= 1
    order = []
    while s.has_work():
        plan, events = run_step(s)
        for e in plan.entries:
            if e.request_id not in order:
                order.append(e.request_id)
        cache.check_invariants()
    assert order == [a, b, c]  # first come, first served
    assert all(s.request(r).state == "completed" for r in (a, b, c))
    assert cache.stats()["kv_pools"]["full"]["used_pages"] == 0
    assert cache.stats()["kv_pools"]["full"]["reserved_pages"] == 0


def test_sequence_limit_and_cancel():
    h = host()
    cache, s = make(h, seqs=2, pages=32)
    p = h.SamplingParams()
    ids = [s.submit([1] * 5, 4, [], p) for _ in range(3)]
    plan, _ = run_step(s)
    assert [e.request_id for e in plan.entries] == ids[:2]
    s.cancel(ids[0])  # mid-run: its pages return at once
    assert s.request(ids[0]).state == "cancelled" and s.request(ids[0]).reason == "cancelled"
    s.cancel(ids[2])  # still waiting
    with pytest.raises(RuntimeError, match="cannot forget an active request"):
        s.forget(ids[1])
    while s.has_work():
        run_step(s)
    assert s.request(ids[1]).state == "completed"
    stats = s.stats()
    assert (stats["submitted"], stats["completed"], stats["cancelled"]) == (3, 1, 2)
    assert cache.stats()["kv_pools"]["full"]["used_pages"] == 0


def test_cancel_between_plan_and_commit_and_abandon():
    h = host()
    cache, s = make(h)
    p = h.SamplingParams()
    a = s.submit([1, 2, 3], 4, [], p)
    b = s.submit([1, 2], 4, [], p)
    plan = s.plan()
    s.cancel(a)
    events = s.commit(plan, [9, 9])
    assert [e.request_id for e in events] == [b]
    plan = s.plan()
    s.abandon(plan)  # the model step threw
    assert s.request(b).state == "cancelled" and s.request(b).reason == "error"
    assert cache.stats()["kv_pools"]["full"]["used_pages"] == 0 and not s.has_work()


def test_draw_keys_follow_the_seed_and_the_step():
    h = host()
    cache, s = make(h)
    a = s.submit([1], 3, [], h.SamplingParams(temperature=0.8, seed=12345))
    b = s.submit([1], 3, [], h.SamplingParams(temperature=0.8))
    assert s.draw_key(a) == (12345 * 1_000_003) % (1 << 63)
    run_step(s)
    assert s.draw_key(a) == (12345 * 1_000_003 + 1) % (1 << 63)
    assert s.draw_key(b) != s.draw_key(a)
    assert not s.request(a).sampling.greedy and h.SamplingParams(temperature=0.8, top_k=1).greedy


def test_when_the_next_step_repeats_this_one():
    """`repeats(plan)`: the next plan is bound to feed the same requests one token each (unless
    a sampled token stops one), which is when the engine may launch that step early."""
    h = host()
    cache, s = make(h, context=40)
    a = s.submit([1] * 5, 8, [], h.SamplingParams())
    plan = s.plan()
    assert not s.repeats(plan)  # a prompt portion
    s.commit(plan, [9])
    plan = s.plan()
    assert [e.decode for e in plan.entries] == [True] and s.repeats(plan)
    s.commit(plan, [9])
    b = s.submit([2] * 3, 20, [], h.SamplingParams())
    plan = s.plan()  # a decodes, b reads its prompt
    assert not s.repeats(plan)
    s.commit(plan, [9, 9])
    plan = s.plan()
    assert [(e.request_id, e.decode) for e in plan.entries] == [(a, True), (b, True)] and s.repeats(plan)
    s.commit(plan, [9, 9])
    following = s.plan()
    assert [(e.request_id, e.start, e.count) for e in following.entries] == [
        (e.request_id, e.start + 1, 1) for e in plan.entries
    ]
    # A forced token and a waiting request say no.
    s.force(a, [3])
    assert not s.repeats(following)
    s.commit(following, [9, 9])
    plan = s.plan()
    assert s.repeats(plan)
    blocked = [s.submit([4] * 3, 2, [], h.SamplingParams()) for _ in range(2)]  # the third sequence, and one that waits
    assert not s.repeats(plan)
    s.commit(plan, [9, 9])
    for r in blocked:
        s.cancel(r)
    # So does the last token before a length limit: a has 6 of its 8 tokens, then 7.
    plan = s.plan()
    assert len(s.request(a).output) == 6 and s.repeats(plan)
    s.commit(plan, [9, 9])
    plan = s.plan()
    assert len(s.request(a).output) == 7 and not s.repeats(plan)
    events = s.commit(plan, [9, 9])
    assert [(e.request_id, e.finished) for e in events] == [(a, True), (b, False)]


def test_repeats_stops_before_the_context_limit():
    h = host()
    cache, s = make(h, context=9)
    a = s.submit([1] * 5, 4, [], h.SamplingParams())  # ends where the context does
    run_step(s)
    plan = s.plan()  # position 5
    assert s.repeats(plan)
    s.commit(plan, [9])
    plan = s.plan()  # position 6
    assert s.repeats(plan)
    s.commit(plan, [9])
    plan = s.plan()  # position 7: this step's token is the last one
    assert not s.repeats(plan)
    events = s.commit(plan, [9])
    assert events[0].finished and not s.has_work()


@pytest.mark.parametrize("seed", range(8))
def test_random_traffic_keeps_every_promise(seed):
    """Random submits, cancels (also between plan and commit) and stop tokens over a full and a
    window group with few pages: every plan keeps the budget, the portion sizes and the order;
    requests start first come, first served; nothing stalls; every page and slot comes back."""
    import numpy as np

    rng = np.random.default_rng(100 + seed)
    h = host()
    page = int(rng.choice([2, 4, 8]))
    window = int(rng.choice([0, 5, 12]))
    seqs = int(rng.integers(1, 5))
    chunk = int(rng.integers(1, 6))
    burst = chunk + int(rng.integers(0, 6))
    budget = seqs + int(rng.integers(0, 9))
    context, vocab = 48, 20
    full_pages = (context + page - 1) // page + int(rng.integers(0, 8))  # the longest request fits, little more
    groups = [h.GroupSpec("full", full_pages, 0)]
    if window:
        groups.append(h.GroupSpec("window", (window + burst + page - 1) // page + 1 + int(rng.integers(0, 4)), window))
    cache = h.CacheManager(page, groups, seqs, burst)
    s = h.Scheduler(cache, seqs, context, budget, chunk, burst, vocab, 1)

    submitted, first_seen, cancelled_waiting, stops = [], [], set(), {}
    steps = 0
    while steps < 400 and (steps < 120 or s.has_work()):
        steps += 1
        if steps < 120 and rng.random() < 0.5:
            prompt = [int(t) for t in rng.integers(0, vocab, int(rng.integers(1, 31)))]
            new = int(rng.integers(1, min(12, context - len(prompt)) + 1))
            stop = [int(rng.integers(0, vocab))] if rng.random() < 0.4 else []
            rid = s.submit(prompt, new, stop, h.SamplingParams())
            submitted.append(rid)
            stops[rid] = set(stop)
        live = [r for r in submitted if s.request(r).state in ("waiting", "prefilling", "running")]
        if live and rng.random() < 0.1:
            victim = int(rng.choice(live))
            if s.request(victim).state == "waiting":
                cancelled_waiting.add(victim)
            s.cancel(victim)
        if not s.has_work():
            continue
        plan = s.plan()
        entries = plan.entries
        assert entries, "work is waiting but the plan is empty"
        assert plan.total_tokens <= budget and len(entries) <= seqs
        assert len({e.request_id for e in entries}) == len(entries)
        kinds = [e.decode for e in entries]
        assert kinds == sorted(kinds, reverse=True), "single decoded tokens come first"
        portion = chunk if any(kinds) else burst
        for e in entries:
            request = s.request(e.request_id)
            assert e.start == cache.length(e.request_id) == request.length
            if e.decode:
                assert e.count == 1 and e.wants_token and request.state == "running"
            else:
                assert 1 <= e.count <= portion and request.state == "prefilling"
                assert e.wants_token == (e.start + e.count == len(request.prompt))
            if e.request_id not in first_seen:
                first_seen.append(e.request_id)
        cache.check_invariants()
        if rng.random() < 0.1:  # a cancel while the step runs
            s.cancel(int(rng.choice([e.request_id for e in entries])))
        events = s.commit(plan, [int(rng.integers(0, vocab)) for e in entries if e.wants_token])
        cache.check_invariants()
        for event in events:
            request = s.request(event.request_id)
            assert len(request.output) <= request.max_new_tokens
            if event.finished:
                assert request.state == "completed" and not cache.contains(event.request_id)
                assert (event.reason == "stop") == (event.token in stops[event.request_id])
                assert event.reason != "length" or len(request.output) == request.max_new_tokens
    assert not s.has_work(), "requests were left over"
    assert first_seen == [r for r in submitted if r in set(first_seen)], "requests started out of order"
    never_started = [r for r in submitted if r not in set(first_seen)]
    assert all(r in cancelled_waiting for r in never_started)
    assert all(s.request(r).state in ("completed", "cancelled") for r in submitted)
    stats = cache.stats()
    for pool in stats["kv_pools"].values():
        assert pool["used_pages"] == 0 and pool["reserved_pages"] == 0
    assert stats["free_state_slots"] == seqs and stats["requests"] == 0
    totals = s.stats()
    assert totals["submitted"] == len(submitted) and totals["completed"] + totals["cancelled"] == len(submitted)
