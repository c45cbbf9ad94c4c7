"""The scheduler's decisions, driven with a fake step function (no device)."""
import hashlib

import pytest

from qwen_decoder_b200.cache import CacheLayout, CacheManager, PagedKV
from qwen_decoder_b200.engine.scheduler import Request, SamplingParams, Scheduler


def manager(num_pages, page_size=16, max_requests=8):
    layout = CacheLayout.from_needs([PagedKV(2, 16), PagedKV(2, 16)], [None, None])
    return CacheManager(layout, num_pages, page_size, max_requests)


def next_token(tokens, vocab=1000):
    """A stand-in model: the next token is a hash of everything before it."""
    h = hashlib.sha256(",".join(map(str, tokens)).encode()).digest()
    return int.from_bytes(h[:4], "little") % vocab


def fake_step(sched, plan):
    """What the engine does with a plan: commit the tokens to the cache, sample where asked."""
    sampled = []
    for e in plan.entries:
        req = e.request
        start = req.num_computed
        assert e.tokens == req.all_tokens()[start:start + len(e.tokens)]
        assert req.cache.num_tokens == start
        sched.cache.commit(req.cache, len(e.tokens))
        if e.samples:
            assert start + len(e.tokens) == len(req.prompt) + len(req.output)
            sampled.append(next_token(req.all_tokens()))
    return sched.update(plan, sampled)


def run(sched, reqs, max_steps=10000):
    for r in reqs:
        sched.add_request(r)
    plans = []
    while sched.has_work():
        plan = sched.schedule()
        plans.append(plan)
        fake_step(sched, plan)
        sched.cache.check()
        assert len(plans) < max_steps
    return plans


def expected_output(prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(next_token(seq))
    return seq[len(prompt):]


def test_prompts_are_cut_under_the_budget_and_decodes_always_run():
    s = Scheduler(manager(200), max_batch=4, max_prefill_tokens_per_step=24, max_total_tokens=64)
    reqs = [Request(i, list(range(1, n + 1)), SamplingParams(max_new_tokens=5)) for i, n in enumerate([30, 10, 50])]
    plans = run(s, reqs)
    # step 0: 24 of request 0; step 1: its last 6, all 10 of request 1, 8 of request 2
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in plans[0].entries] == [(0, 24, False)]
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in plans[1].entries] == \
        [(0, 6, True), (1, 10, True), (2, 8, False)]
    # step 2: requests 0 and 1 decode (first), request 2 goes on with 24 prompt tokens
    assert [(e.request.request_id, len(e.tokens)) for e in plans[2].entries] == [(0, 1), (1, 1), (2, 24)]
    for p in plans:
        prompt_tokens = sum(len(e.tokens) for e in p.entries if not (len(e.tokens) == 1 and e.request.output))
        assert prompt_tokens <= 24
    for r in reqs:
        assert r.finished and r.finish_reason == "length" and r.output == expected_output(r.prompt, 5)
    assert s.cache.free_pages() == [200] and s.cache.slots.num_free == 8
    assert s.stats["prompt_tokens"] == 90 and s.stats["decode_tokens"] == 3 * 4


def test_max_batch_limits_running_and_order_is_fifo():
    s = Scheduler(manager(200), max_batch=2, max_prefill_tokens_per_step=512)
    reqs = [Request(i, [i + 1] * 5, SamplingParams(max_new_tokens=3 + i)) for i in range(5)]
    for r in reqs:
        s.add_request(r)
    seen = []
    while s.has_work():
        plan = s.schedule()
        assert len(s.running) <= 2
        for e in plan.entries:
            if e.request.request_id not in seen:
                seen.append(e.request.request_id)
        fake_step(s, plan)
    assert seen == [0, 1, 2, 3, 4] and all(r.finished for r in reqs)


def test_stop_ids_and_ignore_eos():
    prompt = [3, 1, 4, 1, 5]
    out = expected_output(prompt, 6)
    stop = out[2]
    s = Scheduler(manager(50), stop_ids=[stop])
    a = Request("a", prompt, SamplingParams(max_new_tokens=6))
    b = Request("b", prompt, SamplingParams(max_new_tokens=6, ignore_eos=True))
    c = Request("c", prompt, SamplingParams(max_new_tokens=6, stop_ids=[out[0]]))
    run(s, [a, b, c])
    assert a.finish_reason == "stop" and a.output == out[:2]      # the stop id is not part of the output
    assert b.finish_reason == "length" and b.output == out
    assert c.finish_reason == "stop" and c.output == []


def test_running_out_of_pages_preempts_the_youngest_and_output_is_unchanged():
    # 3 requests start with one page each and grow to 5 pages (10 prompt + 60 new tokens); pool of 9
    def make():
        return [Request(i, [7 * i + j for j in range(10)], SamplingParams(max_new_tokens=60)) for i in range(3)]
    small = Scheduler(manager(9), max_batch=4, max_prefill_tokens_per_step=512)
    reqs = make()
    plans = run(small, reqs)
    assert small.stats["preemptions"] >= 1
    first = next(p for p in plans if p.preempted)
    assert first.preempted[0].request_id == 2                     # the most recently admitted goes first
    for r in reqs:
        assert r.output == expected_output(r.prompt, 60) and r.finish_reason == "length"
    assert reqs[2].preemptions >= 1 and reqs[0].preemptions == 0
    assert small.cache.free_pages() == [9]
    # a preempted request comes back with prompt + what it had generated, and is fed in one go
    back = next(p for p in plans[plans.index(first) + 1:] if any(e.request.request_id == 2 for e in p.entries))
    e = next(e for e in back.entries if e.request.request_id == 2)
    assert len(e.tokens) > 10 and e.tokens[:10] == reqs[2].prompt
    # same plans again: the decisions are deterministic
    again = Scheduler(manager(9), max_batch=4, max_prefill_tokens_per_step=512)
    plans2 = run(again, make())
    assert [[(e.request.request_id, len(e.tokens)) for e in p.entries] for p in plans] == \
           [[(e.request.request_id, len(e.tokens)) for e in p.entries] for p in plans2]


def test_a_request_that_can_never_fit_ends_with_a_reason():
    s = Scheduler(manager(3), max_batch=2)
    big = Request("big", list(range(1, 100)), SamplingParams(max_new_tokens=4))          # 7 pages > 3
    grows = Request("grows", list(range(1, 41)), SamplingParams(max_new_tokens=30))      # 3 pages, then a 4th
    ok = Request("ok", [1, 2, 3], SamplingParams(max_new_tokens=2))
    run(s, [big, grows, ok])
    assert big.finish_reason == "too_long_for_cache" and big.output == []
    assert grows.finish_reason == "too_long_for_cache" and len(grows.output) == 9       # 48 cached tokens fill 3 pages; the 49th cannot be fed
    assert ok.finish_reason == "length" and len(ok.output) == 2
    assert s.cache.free_pages() == [3]


def test_max_positions_ends_a_request():
    s = Scheduler(manager(50), max_positions=12)
    a = Request("a", list(range(1, 9)), SamplingParams(max_new_tokens=100))
    b = Request("b", list(range(1, 20)), SamplingParams(max_new_tokens=1))
    run(s, [a, b])
    assert a.finish_reason == "max_positions" and len(a.prompt) + len(a.output) == 12
    assert b.finish_reason == "too_long"


def test_prefix_cache_skips_known_beginnings_and_keeps_the_output():
    layout = CacheLayout.from_needs([PagedKV(2, 16)], [None])

    def run_with(prefix):
        cache = CacheManager(layout, 64, 16, 8, prefix_cache=prefix)
        s = Scheduler(cache, max_batch=2, max_prefill_tokens_per_step=512)
        stem = list(range(1, 41))
        reqs = [Request(i, stem + [100 + i, 200 + i], SamplingParams(max_new_tokens=4)) for i in range(4)]
        for r in reqs:
            s.add_request(r)
        while s.has_work():
            plan = s.schedule()
            sampled = []
            for e in plan.entries:
                req = e.request
                assert e.tokens == req.all_tokens()[req.num_computed:req.num_computed + len(e.tokens)]
                cache.commit(req.cache, len(e.tokens), e.tokens)
                if e.samples:
                    sampled.append(next_token(req.all_tokens()))
            s.update(plan, sampled)
            cache.check()
        return reqs, s

    plain, s0 = run_with(False)
    cached, s1 = run_with(True)
    assert [r.output for r in plain] == [r.output for r in cached]
    assert s0.stats["prompt_tokens"] == 4 * 42
    # requests 2 and 3 start after 0 and 1 have cached the 32 tokens of the stem's two full pages
    assert s1.stats["prefix_hit_tokens"] >= 2 * 32 and s1.stats["prompt_tokens"] == 4 * 42 - s1.stats["prefix_hit_tokens"]
    assert s1.cache.free_pages() == [64]


def test_prefix_hit_in_a_nearly_full_pool_waits_instead_of_failing():
    """A known beginning takes its pages off the free list when the request is opened: the room check has
    to count what is free after that.  Pool of 256 pages; a finished request left 200 recorded pages on
    the free list; a running request holds 30; a request with the recorded beginning plus 512 tokens
    then finds 26 free pages where its first portion needs 32: it must wait, not raise."""
    layout = CacheLayout.from_needs([PagedKV(2, 16)], [None])
    cache = CacheManager(layout, 256, 16, 8, prefix_cache=True)
    s = Scheduler(cache, max_batch=4, max_prefill_tokens_per_step=512, max_total_tokens=1024)

    def step():
        plan = s.schedule()
        sampled = []
        for e in plan.entries:
            cache.commit(e.request.cache, len(e.tokens), e.tokens)
            if e.samples:
                sampled.append(next_token(e.request.all_tokens()))
        s.update(plan, sampled)
        cache.check()
        return plan

    stem = [(7 * i) % 991 + 1 for i in range(3200)]
    first = Request("first", stem + [5], SamplingParams(max_new_tokens=1))
    s.add_request(first)
    while s.has_work():
        step()
    assert first.finished and cache.free_pages() == [256]
    holder = Request("holder", [900 - (i % 50) for i in range(30 * 16 - 8)], SamplingParams(max_new_tokens=1000))
    s.add_request(holder)
    step()
    assert len(holder.cache.tables[0]) == 30
    again = Request("again", stem + [(11 * i) % 977 + 1 for i in range(512)], SamplingParams(max_new_tokens=2))
    s.add_request(again)
    plan = step()                        # would raise OutOfPages out of schedule() before
    assert again.cache is None and list(s.waiting) == [again] and "again" not in cache.live
    assert [e.request for e in plan.entries] == [holder]
    assert cache.free_pages() == [256 - 30]
    # once the holder is gone the request runs, and finds its beginning
    s._finish(holder, "cancelled")
    while s.has_work():
        step()
    assert again.finished and again.finish_reason == "length" and len(again.output) == 2
    assert s.stats["prefix_hit_tokens"] >= 3200 and cache.free_pages() == [256]


def run_ahead(sched, reqs, max_steps=10000):
    """The engine's pipelined loop with a fake step: a step's sampled tokens are handed to ``update`` only
    after the next step has been planned (``plan_ahead``) and committed."""
    for r in reqs:
        sched.add_request(r)
    ahead_steps = usual_steps = 0
    in_flight = None                      # (plan, sampled tokens not yet given to update)

    def launch(plan, ahead):
        sampled = []
        for e in plan.entries:
            req = e.request
            # what the cache holds after the tokens of this step: known from the cache alone
            sched.cache.commit(req.cache, len(e.tokens))
            if e.samples:
                known = req.all_tokens() + ([pending[req.request_id]] if ahead else [])
                sampled.append(next_token(known))
        return plan, sampled

    pending = {}
    while sched.has_work() or in_flight is not None:
        if in_flight is None:
            plan = sched.schedule()
            if not plan.entries:
                continue
            in_flight = launch(plan, False)
            usual_steps += 1
        plan, sampled = in_flight
        in_flight = None
        pending = {e.request.request_id: t for e, t in zip([e for e in plan.entries if e.samples], sampled)}
        nxt = sched.plan_ahead(plan)
        if nxt is not None:
            in_flight = launch(nxt, True)
            ahead_steps += 1
        sched.update(plan, sampled)
        sched.cache.check()
        assert ahead_steps + usual_steps < max_steps
    return usual_steps, ahead_steps


def test_planning_ahead_gives_the_same_output_and_stops_where_it_must():
    def requests():
        return [Request(i, list(range(1, n + 1)), SamplingParams(max_new_tokens=m, ignore_eos=True))
                for i, (n, m) in enumerate([(30, 12), (10, 40), (50, 25)])]
    a = requests()
    usual, ahead = run_ahead(Scheduler(manager(200), max_batch=4, max_prefill_tokens_per_step=24), a)
    for r in a:
        assert r.output == expected_output(r.prompt, r.params.max_new_tokens) and r.finish_reason == "length"
    assert ahead > usual          # most decode steps were planned before their tokens were known
    # a stop token ends a request one step late for the device, never for the output
    probe = Request(0, [5, 6, 7], SamplingParams(max_new_tokens=30, ignore_eos=True))
    run(Scheduler(manager(50)), [probe])
    stop = probe.output[9]
    b = [Request(0, [5, 6, 7], SamplingParams(max_new_tokens=30, stop_ids=[stop])),
         Request(1, [9, 9, 9, 9], SamplingParams(max_new_tokens=30, ignore_eos=True))]
    s = Scheduler(manager(50))
    run_ahead(s, b)
    assert b[0].finish_reason == "stop" and b[0].output == probe.output[:probe.output.index(stop)]
    assert b[1].output == expected_output(b[1].prompt, 30)
    assert s.cache.free_pages() == [50] and not s.cache.live


def test_planning_ahead_declines_when_the_usual_path_has_to_decide():
    s = Scheduler(manager(4, page_size=16), max_batch=4)
    r0 = Request(0, list(range(1, 31)), SamplingParams(max_new_tokens=40, ignore_eos=True))
    s.add_request(r0)
    plan = s.schedule()
    for e in plan.entries:
        s.cache.commit(e.request.cache, len(e.tokens))
    # the plan fed a prompt of several tokens: entries are not single decoded tokens
    assert s.plan_ahead(plan) is None
    s.update(plan, [7])
    plan = s.schedule()
    s.cache.commit(r0.cache, 1)
    # somebody waits: admission is the usual path's business
    s.add_request(Request(1, [1, 2, 3], SamplingParams(max_new_tokens=4)))
    assert s.plan_ahead(plan) is None
    s.waiting.clear()
    ahead = s.plan_ahead(plan)
    assert ahead is not None and [e.request for e in ahead.entries] == [r0]
    s.update(plan, [8])
    # out of pages: 4 pages of 16 hold 64 tokens; at 64 cached tokens the next one needs a fifth page
    while r0.cache.num_tokens < 63:
        s.cache.commit(r0.cache, 1)
        s.update(ahead, [9])
        ahead = s.plan_ahead(ahead) or ahead
    s.cache.commit(r0.cache, 1)
    assert r0.cache.num_tokens == 64 and s.plan_ahead(ahead) is None
    # the last token of a request: the usual path ends it
    s2 = Scheduler(manager(20))
    r = Request(0, [1, 2, 3], SamplingParams(max_new_tokens=2, ignore_eos=True))
    s2.add_request(r)
    p = s2.schedule(); s2.cache.commit(r.cache, 3); s2.update(p, [4])
    p = s2.schedule(); s2.cache.commit(r.cache, 1)
    assert s2.plan_ahead(p) is None


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_random_arrivals_keep_every_rule(seed):
    """Requests of random lengths arriving while others run, in a pool small enough to force preemption:
    every plan keeps the budgets, every request ends with the output it would have had alone, and the pool
    is whole again at the end."""
    import random
    rng = random.Random(seed)
    budget, total, max_batch = rng.choice([16, 24, 40]), 48, rng.choice([2, 3, 5])
    cache = manager(rng.choice([10, 14, 24]), page_size=16, max_requests=max_batch)
    s = Scheduler(cache, max_batch=max_batch, max_prefill_tokens_per_step=budget, max_total_tokens=total)
    specs = [([rng.randrange(1000) for _ in range(rng.randint(1, 70))], rng.randint(1, 30)) for _ in range(12)]
    reqs = [Request(i, p, SamplingParams(max_new_tokens=n, ignore_eos=True)) for i, (p, n) in enumerate(specs)]
    waiting = list(reqs)
    steps = 0
    while waiting or s.has_work():
        for _ in range(rng.randint(0, 2)):
            if waiting:
                s.add_request(waiting.pop(0))
        if not s.has_work():
            continue
        plan = s.schedule()
        portions = [e for e in plan.entries if len(e.tokens) > 1]
        assert sum(len(e.tokens) for e in portions) <= budget
        assert sum(len(e.tokens) for e in plan.entries) <= total
        assert len({id(e.request) for e in plan.entries}) == len(plan.entries) <= max_batch
        fake_step(s, plan)
        cache.check()
        steps += 1
        assert steps < 5000
    for r, (p, n) in zip(reqs, specs):
        if r.finish_reason == "too_long_for_cache":          # could never fit this pool, even alone
            assert (len(p) + n + 15) // 16 > cache.num_pages
            continue
        assert r.output == expected_output(p, n), (r.request_id, r.finish_reason)
    assert cache.free_pages() == [cache.num_pages] * len(cache.pools)
