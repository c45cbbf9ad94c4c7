"""Continuous batching: admit requests, cut prompts into portions under a token
budget, decode, finish and free.  Host-only: it plans steps and is told their results;
it never touches the device, so it can be driven with a fake step function.

What it keeps from the reference (scheduler.h:35-110, scheduler.cpp:5-86,
decoder.cpp:35-239): a FIFO waiting queue and at most ``max_batch`` running requests
(scheduler.cpp:16-41); per step a shared prompt-token budget
``max_prefill_tokens_per_step`` handed out in admission order, each prefilling request
taking min(remaining, budget) (decoder.cpp:90-96,129), while every decoding request
always gets its one token (decoder.cpp:130-157); pages are taken lazily as the cached
length grows (scheduler.cpp:67-80); the step that consumes the last prompt token
samples the first new token (decoder.cpp:208-211); finished requests give their
pages back at the end of the step (decoder.cpp:236).

What it decides differently: when pages run out the reference marks the request
finished and drops it (scheduler.cpp:72-76, decoder.cpp:106-109).  Here the most
recently admitted running request is *preempted*: its pages and state slot are given
back and it returns to the front of the waiting queue with prompt + generated tokens
to be recomputed.  A request that cannot fit in the pool even alone ends with the
reason ``too_long_for_cache``.  New requests are admitted only while the pool has room
for their first portion.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence

from ..cache import CacheManager, OutOfPages, RequestCache


@dataclass
class SamplingParams:
    """Defaults follow the reference's main (gpu_main.cu:45-48) except top_k, which is off."""
    temperature: float = 0.0
    top_k: int = 0
    max_new_tokens: int = 256
    seed: int = 0
    stop_ids: Sequence[int] = ()
    ignore_eos: bool = False


@dataclass
class Request:
    request_id: object
    prompt: List[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    output: List[int] = field(default_factory=list)
    cache: Optional[RequestCache] = None
    num_computed: int = 0             # tokens of prompt + output whose cache entries exist
    finished: bool = False
    finish_reason: Optional[str] = None
    preemptions: int = 0
    admitted_at: int = -1             # admission counter, for the preemption order

    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def num_pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.num_computed


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    samples: bool                     # this portion ends with the request's last known token


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    finished: List[Request] = field(default_factory=list)     # ended while planning (cannot fit)

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch: int = 64, max_prefill_tokens_per_step: int = 512,
                 max_total_tokens: int = 4096, max_positions: int = 1 << 30, stop_ids: Sequence[int] = ()):
        if max_batch < 1 or max_prefill_tokens_per_step < 1:
            raise ValueError("max_batch and max_prefill_tokens_per_step must be at least 1")
        self.cache = cache
        self.max_batch = min(max_batch, cache.max_requests)
        self.max_prefill_tokens_per_step = max_prefill_tokens_per_step
        # as gpu_decoder.cu:168: room for a full prompt budget beside every decode token
        self.max_total_tokens = max(max_total_tokens, max_prefill_tokens_per_step + self.max_batch)
        self.max_positions = max_positions
        self.default_stop_ids = tuple(stop_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._admissions = 0
        self.stats = {"steps": 0, "prompt_tokens": 0, "decode_tokens": 0, "preemptions": 0, "finished": 0}

    # ---- queueing --------------------------------------------------------
    def add_request(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError(f"request {req.request_id!r}: empty prompt")
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- planning ----------------------------------------------------------
    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self.cache.close(req.cache)
        req.cache = None
        req.num_computed = 0
        req.preemptions += 1
        self.running.remove(req)
        self.waiting.appendleft(req)
        plan.preempted.append(req)
        plan.entries = [e for e in plan.entries if e.request is not req]
        self.stats["preemptions"] += 1

    def _finish(self, req: Request, reason: str) -> None:
        req.finished = True
        req.finish_reason = reason
        if req.cache is not None:
            self.cache.close(req.cache)
            req.cache = None
        if req in self.running:
            self.running.remove(req)
        self.stats["finished"] += 1

    def _take_pages(self, req: Request, n: int, plan: StepPlan) -> bool:
        """Pages for ``n`` more tokens of ``req``, preempting later-admitted requests if needed.
        False if ``req`` itself had to go."""
        while True:
            try:
                self.cache.ensure(req.cache, req.num_computed + n)
                return True
            except OutOfPages:
                victim = max(self.running, key=lambda r: r.admitted_at)
                if victim is req and len(self.running) == 1:
                    # alone and still too big: it can never run
                    self._finish(req, "too_long_for_cache")
                    plan.finished.append(req)
                    plan.entries = [e for e in plan.entries if e.request is not req]
                    return False
                self._preempt(victim, plan)
                if victim is req:
                    return False

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        budget = self.max_total_tokens
        prompt_budget = self.max_prefill_tokens_per_step
        # 1. every decoding request gets its token (oldest first, so the youngest are preempted)
        for req in sorted(self.running, key=lambda r: r.admitted_at):
            if req not in self.running or req.num_pending != 1 or not req.output:
                continue
            if self._take_pages(req, 1, plan):
                plan.entries.append(PlannedEntry(req, [req.output[-1]], True))
                budget -= 1
        # 2. running requests that still have several tokens to feed, in admission order
        for req in sorted(self.running, key=lambda r: r.admitted_at):
            if req not in self.running or any(e.request is req for e in plan.entries):
                continue
            n = min(req.num_pending, prompt_budget, budget)
            if n <= 0:
                continue
            if self._take_pages(req, n, plan):
                toks = req.all_tokens()[req.num_computed:req.num_computed + n]
                plan.entries.append(PlannedEntry(req, toks, n == req.num_pending))
                prompt_budget -= n
                budget -= n
        # 3. admit waiting requests while there is a slot, budget and room for a first portion
        while self.waiting and len(self.running) < self.max_batch and prompt_budget > 0 and budget > 0 \
                and not plan.preempted:
            req = self.waiting[0]
            total = len(req.prompt) + len(req.output)
            if total > self.max_positions:
                self.waiting.popleft()
                self._finish(req, "too_long")
                plan.finished.append(req)
                continue
            ps = self.cache.page_size
            if any((total + ps - 1) // ps > pool.num_pages for pool in self.cache.pools):
                self.waiting.popleft()          # would not fit even alone
                self._finish(req, "too_long_for_cache")
                plan.finished.append(req)
                continue
            if self.cache.slots.num_free == 0:
                break
            tokens = req.all_tokens()
            # Open first: with the prefix cache a known beginning takes its pages off the free list, so the
            # room that counts is what is free afterwards.  Room for the first portion, and one page of
            # growth for every running request; if it is not there the request goes back where it was.
            rc = self.cache.open(req.request_id, tokens)
            n = min(total - rc.num_tokens, prompt_budget, budget)
            missing = self.cache.pages_missing(rc, rc.num_tokens + n)
            if any(m + len(self.running) > free for m, free in zip(missing, self.cache.free_pages())):
                self.cache.close(rc)
                break
            self.waiting.popleft()
            req.cache = rc
            req.num_computed = rc.num_tokens
            req.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(req)
            self.cache.ensure(rc, req.num_computed + n)
            self.stats["prefix_hit_tokens"] = self.stats.get("prefix_hit_tokens", 0) + req.num_computed
            plan.entries.append(PlannedEntry(req, tokens[req.num_computed:req.num_computed + n],
                                             req.num_computed + n == total))
            prompt_budget -= n
            budget -= n
        return plan

    def plan_ahead(self, plan: StepPlan) -> Optional[StepPlan]:
        """The step after ``plan``, planned before ``plan``'s sampled tokens are known: possible when
        ``plan`` is one decoded token for every running request, nobody waits, and no request can be
        seen to end with it.  The entries' tokens are placeholders (the step function takes them from
        the device); a request that ends with ``plan`` after all (a stop token) keeps its entry and
        ``update`` skips it.  None if the next step has to be planned the usual way."""
        if self.waiting or not plan.entries or plan.preempted or len(plan.entries) != len(self.running):
            return None
        for e in plan.entries:
            r = e.request
            if len(e.tokens) != 1 or not e.samples or r.cache is None:
                return None
            if len(r.output) + 1 >= r.params.max_new_tokens or \
                    len(r.prompt) + len(r.output) + 1 >= self.max_positions:
                return None                  # its last token: the usual path ends it
        ahead = StepPlan()
        try:
            for e in plan.entries:
                self.cache.ensure(e.request.cache, e.request.cache.num_tokens + 1)
                ahead.entries.append(PlannedEntry(e.request, [0], True))
        except OutOfPages:
            return None                      # the usual path decides whom to preempt
        return ahead

    # ---- results -----------------------------------------------------------
    def _stops(self, req: Request, token: int) -> bool:
        if req.params.ignore_eos:
            return False
        return token in req.params.stop_ids or token in self.default_stop_ids

    def update(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """The step ran; ``sampled`` holds one token per entry with ``samples`` set, in order.
        Returns the requests that finished."""
        done: List[Request] = []
        it = iter(sampled)
        self.stats["steps"] += 1
        for e in plan.entries:
            req = e.request
            if req.finished:               # planned ahead, and the step before ended it
                if e.samples:
                    next(it, None)
                continue
            n = len(e.tokens)
            req.num_computed += n          # the step function has committed them to the cache
            if n == 1 and req.output and e.samples:
                self.stats["decode_tokens"] += 1
            else:
                self.stats["prompt_tokens"] += n
            if not e.samples:
                continue
            token = int(next(it))
            if self._stops(req, token):
                self._finish(req, "stop")
                done.append(req)
                continue
            req.output.append(token)
            if len(req.output) >= req.params.max_new_tokens:
                self._finish(req, "length")
                done.append(req)
            elif len(req.prompt) + len(req.output) >= self.max_positions:
                self._finish(req, "max_positions")
                done.append(req)
        return done
