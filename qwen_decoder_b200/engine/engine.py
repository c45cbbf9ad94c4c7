"""The Python entry point: ``Engine(model_dir, ...)`` and ``generate``.

Option names and meanings are the reference's where it has them: ``max_batch``,
``max_prefill_len``, ``max_prefill_tokens_per_step`` (its command line's
max_prefill_step) and ``max_total_tokens`` are GPUDecoder's constructor arguments
(gpu_decoder.h:72-75, gpu_main.cu:19-34); ``max_new_tokens``, ``temperature`` and
``top_k`` are generate_continuous's (decoder.h:148-154).  Prompts are lists of token
ids: the engine starts at token ids and ends at token ids (the reference's tokenizer,
common.cpp:229-562, is outside it).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence

import torch

from ..cache import CacheManager
from ..sampling import Sampler, uniform_draw
from .batch import StepEntry
from .runner import ModelRunner, resolve_dtype
from .scheduler import Request, SamplingParams, Scheduler, StepPlan


class Engine:
    def __init__(self, model=None, *, config=None, random_seed: Optional[int] = None, dtype="bfloat16",
                 device="cuda:0", max_batch: int = 64, max_prefill_len: int = 4096,
                 max_prefill_tokens_per_step: int = 512, max_total_tokens: int = 4096,
                 page_size: int = 16, num_pages: Optional[int] = None, kv_memory_fraction: float = 0.8,
                 max_positions: Optional[int] = None, use_graphs: bool = True,
                 enable_prefix_cache: bool = False, run_ahead: bool = True, record_steps: bool = False):
        """``model``: a folder with config.json and model.safetensors; or give ``config`` (a typed
        configuration) and ``random_seed`` for random weights made on the device.

        ``max_batch``: most requests running at once.  ``max_prefill_len``: longest prompt taken
        (longer prompts end with ``too_long``; the reference stores this number and never uses it,
        gpu_decoder.h:113-119).  ``max_prefill_tokens_per_step``: prompt tokens per step, shared by
        all prefilling requests.  ``max_total_tokens``: most tokens in one step.  ``num_pages``:
        cache pages of ``page_size`` tokens; by default ``kv_memory_fraction`` of the free device
        memory after the weights, as the reference takes 80 % (gpu_decoder.cu:197-204).
        ``enable_prefix_cache``: requests whose prompts begin alike share the full pages of the common
        part (the reference's generate_continuous argument, decoder.h:148-154).
        ``run_ahead``: while a decode step runs on the device, the next one is already planned and
        launched with the tokens it needs taken from the device; the host reads a step's tokens one
        step late.  The tokens are the same; a request that ends on a stop token costs one wasted row.
        ``record_steps``: keep one record per step (``step_records()``): tokens, how many of them prompt and
        decoded tokens, requests, device time by CUDA events, free pages, queue lengths -- what the reference
        prints per step (decoder.cpp:178-185) and more; each step is also an NVTX range then."""
        self.max_prefill_len = max_prefill_len
        make = dict(dtype=dtype, device=device, page_size=page_size, max_requests=max_batch,
                    max_positions=max_positions, use_graphs=use_graphs, prefix_cache=enable_prefix_cache)
        sizing = _PageSizing(num_pages, kv_memory_fraction, page_size, resolve_dtype(dtype))
        if model is not None:
            self.runner = ModelRunner.from_folder(model, num_pages=sizing, **make)
        elif config is not None:
            self.runner = ModelRunner.from_random(config, seed=random_seed or 0, num_pages=sizing, **make)
        else:
            raise ValueError("give a model folder, or config= and random_seed=")
        self.config = self.runner.config
        self.device = self.runner.device
        self.scheduler = Scheduler(self.runner.cache, max_batch=max_batch,
                                   max_prefill_tokens_per_step=max_prefill_tokens_per_step,
                                   max_total_tokens=max_total_tokens,
                                   max_positions=self.runner.max_positions,
                                   stop_ids=getattr(self.config, "eos_token_ids", ()))
        self.runner.max_step_tokens = self.scheduler.max_total_tokens
        self._next_id = 0
        self._keys: Dict[int, int] = {}
        self.run_ahead = run_ahead
        self._in_flight: Optional[_InFlight] = None      # a launched step whose tokens are not read yet
        self._host_tokens = [torch.empty(self.scheduler.max_batch, dtype=torch.int32, pin_memory=True)
                             for _ in range(2)]
        self._turn = 0
        self._records: Optional[list] = [] if record_steps else None

    # ---- streaming use -----------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id=None) -> Request:
        rid = self._next_id if request_id is None else request_id
        self._next_id += 1
        req = Request(rid, [int(t) for t in prompt], params or SamplingParams())
        req.sample_key = self._next_id - 1
        if len(req.prompt) > self.max_prefill_len:
            req.finished, req.finish_reason = True, "too_long"
            return req
        self.scheduler.add_request(req)
        return req

    def has_work(self) -> bool:
        return self._in_flight is not None or self.scheduler.has_work()

    def _launch(self, plan: StepPlan, device_tokens=None) -> "_InFlight":
        """Run ``plan``'s step; its sampled tokens start their way to a pinned host buffer."""
        entries = [StepEntry(e.request.cache, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                   for e in plan.entries]
        sampling = [e.request for e in plan.entries if e.samples]
        flight = _InFlight(plan, len(sampling), device_tokens is not None)
        rec = self._begin_record(plan, device_tokens is not None)
        if not sampling:
            self.runner.step(entries, ensure_pages=False)
            self._end_record(rec)
            return flight
        ahead = 1 if device_tokens is not None else 0       # a step planned ahead samples one token later
        _, ids = self.runner.step(entries, ensure_pages=False, device_tokens=device_tokens, sampling=(
            [r.params.temperature for r in sampling], [r.params.top_k for r in sampling],
            [uniform_draw(r.params.seed, r.sample_key, len(r.output) + ahead) if r.params.temperature else 0.0
             for r in sampling]))
        self._end_record(rec)
        self._turn ^= 1
        flight.host = self._host_tokens[self._turn][:len(sampling)]
        flight.host.copy_(ids, non_blocking=True)
        flight.event = torch.cuda.Event()
        flight.event.record()
        flight.device = ids
        return flight

    def step(self) -> List[Request]:
        """Plan one step, run it, sample, and return the requests that finished in it.  With
        ``run_ahead`` the step whose results are returned was launched by the call before, and this
        call launches the next one before it waits."""
        finished: List[Request] = []
        cur = self._in_flight
        self._in_flight = None
        if cur is None:
            plan = self.scheduler.schedule()
            finished = list(plan.finished)
            if not plan.entries:
                return finished
            cur = self._launch(plan)
        if self.run_ahead and cur.n_samples == len(cur.plan.entries) and cur.device is not None:
            entries = [StepEntry(e.request.cache, [0], [0]) for e in cur.plan.entries]
            if self.runner.can_take_device_tokens(entries):
                ahead = self.scheduler.plan_ahead(cur.plan)
                if ahead is not None:
                    self._in_flight = self._launch(ahead, device_tokens=cur.device)
        tokens: List[int] = []
        if cur.n_samples:
            cur.event.synchronize()
            tokens = cur.host.tolist()
        if self._in_flight is not None:
            # the step launched ahead feeds exactly these tokens: now the prefix cache may know them
            for e, t in zip(cur.plan.entries, tokens):
                if e.request.cache is not None:
                    self.runner.cache.log_tokens(e.request.cache, [t])
        finished += self.scheduler.update(cur.plan, tokens)
        if finished:
            self.runner.check_status()       # before results leave: no kernel's wait ran out on the way
        return finished

    # ---- batch use -----------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[List[int]]:
        """Generate for every prompt (token ids in, token ids out), continuous batching inside.
        ``params``: one SamplingParams for all, or one per prompt."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.has_work():
            self.step()
        self.runner.check_status()
        return [r.output for r in reqs]

    # ---- per-step records ------------------------------------------------------
    def _begin_record(self, plan: StepPlan, ahead: bool) -> Optional[dict]:
        if self._records is None:
            return None
        decode = sum(1 for e in plan.entries if len(e.tokens) == 1 and e.request.output)
        rec = {"step": len(self._records), "tokens": plan.num_tokens, "decode_tokens": decode,
               "prompt_tokens": plan.num_tokens - decode, "requests": len(plan.entries),
               "prompt_requests": len(plan.entries) - decode, "planned_ahead": ahead,
               "preempted": len(plan.preempted), "running": len(self.scheduler.running),
               "waiting": len(self.scheduler.waiting), "pages_free": self.runner.cache.free_pages(),
               "_events": (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))}
        torch.cuda.nvtx.range_push(f"step {rec['step']}: {rec['prompt_tokens']} prompt + {decode} decode tokens")
        rec["_events"][0].record()
        return rec

    def _end_record(self, rec: Optional[dict]) -> None:
        if rec is None:
            return
        rec["_events"][1].record()
        torch.cuda.nvtx.range_pop()
        self._records.append(rec)

    def step_records(self) -> List[dict]:
        """The records kept with ``record_steps`` (device times read now: waits for the last recorded step)."""
        out = []
        for rec in self._records or []:
            if "_events" in rec:
                e0, e1 = rec.pop("_events")
                e1.synchronize()
                rec["ms"] = round(e0.elapsed_time(e1), 4)
            out.append(rec)
        return out

    @property
    def stats(self) -> dict:
        return dict(self.scheduler.stats, model_steps=self.runner.steps, model_tokens=self.runner.tokens_run)


class _InFlight:
    """A launched step: its plan, and where its sampled tokens arrive."""

    def __init__(self, plan: StepPlan, n_samples: int, ahead: bool):
        self.plan = plan
        self.n_samples = n_samples
        self.ahead = ahead
        self.host: Optional[torch.Tensor] = None       # pinned; valid once ``event`` has passed
        self.event: Optional[torch.cuda.Event] = None
        self.device: Optional[torch.Tensor] = None     # the same tokens on the device


class _PageSizing:
    """How many pages the pool gets: a number, or a share of the memory left after the weights."""

    def __init__(self, num_pages, fraction, page_size, dtype):
        self.num_pages, self.fraction, self.page_size, self.dtype = num_pages, fraction, page_size, dtype

    def resolve(self, layout, device, max_requests, max_positions) -> int:
        if self.num_pages is not None:
            return int(self.num_pages)
        free, _ = torch.cuda.mem_get_info(device)
        per_page = max(1, CacheManager.bytes_per_page(layout, self.page_size, self.dtype))
        by_memory = int(free * self.fraction) // per_page
        # no more than every request at full length could use
        useful = max_requests * ((max_positions + self.page_size - 1) // self.page_size)
        return max(1, min(by_memory, useful))
