"""The step function: a batch of (request, its next tokens) in, logits at the wanted
places out.  It runs only the tokens it is given, as one flat batch, reading earlier
tokens from the cache; portions of prompts and single decoded tokens mix freely.

This is the flat form of the reference's forward_flat + update_block_table_partial +
get_logits_batch (decoder.h:53-77; gpu_decoder.cu:232-542).  Generation
(``engine.Engine``), trace replay (``engine.trace``) and the benchmarks all call this
one function.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..cache import CacheManager, RequestCache
from ..config import describe_model, load_config
from ..parts.model import DecoderModel, build_model
from ..weights import TensorSource, load_into, random_tensors
from .batch import MetaLayout, StepEntry, StepError, build_context, fill, validate

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32,
          "fp32": torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"engine dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"engine dtype must be 'bfloat16' or 'float32', got {dtype!r}") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("the engine runs on a CUDA device only: there is no CPU path "
                           f"(asked for {device}, torch.cuda.is_available() = {torch.cuda.is_available()})")
    return device


class ModelRunner:
    """A bound model, its cache, and ``step``."""

    def __init__(self, model: DecoderModel, config, num_pages: int, page_size: int = 16,
                 max_requests: int = 64, max_positions: Optional[int] = None, use_graphs: bool = True,
                 prefix_cache: bool = False, max_step_tokens: Optional[int] = None):
        self.model = model
        self.config = config
        self.device = model.device
        self.dtype = model.dtype
        self.layout = model.cache_layout()
        model.prepare(max_positions or model.max_positions)
        self.max_positions = model.prepared_positions
        if hasattr(num_pages, "resolve"):      # sized from the memory left after the weights
            num_pages = num_pages.resolve(self.layout, self.device, max_requests, self.max_positions)
        self.cache = CacheManager(self.layout, num_pages, page_size, max_requests, dtype=self.dtype,
                                  device=self.device, prefix_cache=prefix_cache)
        from ..sampling import Sampler
        self.sampler = Sampler(self.device)
        # decode steps replay as CUDA graphs unless a part has to see the step's metadata on the host
        self.use_graphs = use_graphs and not any(
            getattr(part, "needs_host_metadata", False) for part in model.all_parts())
        self.max_step_tokens = max_step_tokens     # most tokens one step may hold (None: no limit of its own)
        self._graphs = {}
        self.steps = 0
        self.tokens_run = 0

    STATUS_EVERY = 512       # steps between two routine looks at the kernels' status words (each look synchronises)

    # ---- construction ----------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda:0", **kw) -> "ModelRunner":
        device = require_cuda(device)
        dt = resolve_dtype(dtype)
        config = load_config(model_dir)
        model = build_model(describe_model(config))
        load_into(model, TensorSource.from_folder(model_dir), dt, device)
        return cls(model, config, **kw)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", **kw) -> "ModelRunner":
        """Random weights made on the device (no folder); same distributions as ``write_random_model``."""
        device = require_cuda(device)
        dt = resolve_dtype(dtype)
        model = build_model(describe_model(config))
        specs = {s.name: s for s in model.tensor_specs()}
        from ..weights.random_init import random_tensor
        src = TensorSource(lambda n: random_tensor(specs[n], seed, torch.bfloat16, device),
                           {n: tuple(s.shape) for n, s in specs.items()}, "random weights")
        load_into(model, src, dt, device)
        return cls(model, config, **kw)

    # ---- requests ----------------------------------------------------------
    def open(self, request_id, tokens=None) -> RequestCache:
        return self.cache.open(request_id, tokens)

    def close(self, rc: RequestCache) -> None:
        self.cache.close(rc)

    # ---- the step ------------------------------------------------------------
    def _ensure(self, entries: Sequence[StepEntry]) -> None:
        taken = []
        try:
            for e in entries:
                before = [len(t) for t in e.cache.tables]
                taken.append((e.cache, before))
                self.cache.ensure(e.cache, e.cache.num_tokens + len(e.tokens))
        except Exception:
            for rc, before in taken:     # all or nothing over the whole batch
                for g, table in enumerate(rc.tables):
                    while len(table.pages) > before[g]:
                        self.cache.pools[g].release(table.pages.pop())
            raise

    def step(self, entries: Sequence[StepEntry], ensure_pages: bool = True, sampling=None,
             device_tokens: Optional[torch.Tensor] = None):
        """Run one batch; returns float32 logits [wanted places in entry order, vocab] on the device.

        With ``ensure_pages`` the pages the new tokens need are taken first (``OutOfPages`` if the
        pool cannot give them; nothing is taken then).  Afterwards each request's cached length has
        grown by its tokens.  With ``sampling`` = (temperatures, top_ks, draws), one per wanted
        place, returns (logits, sampled int32 tokens on the device).

        ``device_tokens`` (int32 on the device, one per entry): the entries' single tokens are not known
        on the host yet -- they are what an earlier step sampled and has not been read back -- and are
        taken from there; the entries' own token values are ignored and the prefix cache is told later
        (``cache.log_tokens``).  Only for batches that run as a graph (``can_take_device_tokens``).

        A batch of single tokens that all want logits runs as a replayed CUDA graph (one per padded
        batch size and block-table width) when ``use_graphs`` is set; the logits then live in a
        buffer that the next such step overwrites."""
        if ensure_pages:
            self._ensure(entries)
        if self.can_take_device_tokens(entries):
            logits, tokens = self._graph_step(entries, sampling, device_tokens)
            n_tokens = len(entries)
        elif device_tokens is not None:
            raise StepError("device_tokens: only a batch of single tokens that all want logits takes them")
        else:
            from .. import kernels
            ctx = build_context(entries, self.cache, self.device, self.model.vocab_size, self.max_positions,
                                self.max_step_tokens)
            with kernels.step_stream():
                logits = self.model.forward(ctx)
                tokens = None
                if sampling is not None and ctx.num_wanted:
                    tokens = self.sampler.sample(logits, *sampling)
            n_tokens = ctx.num_tokens
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens), e.tokens if device_tokens is None else None)
        self.steps += 1
        self.tokens_run += n_tokens
        if self.steps % self.STATUS_EVERY == 0:
            self.check_status()          # a wait inside a kernel that ran out must not pass unnoticed
        return logits if sampling is None else (logits, tokens)

    def check_status(self) -> None:
        """Raise ``KernelError`` if a bounded wait inside a kernel ran out since the last look: what the
        steps since then returned is void.  Synchronises the device.  Callers look before they hand
        results out: ``Engine`` whenever requests finish, trace replay after every step that writes
        logits, and every ``STATUS_EVERY`` steps in between.  After a fault the parts put the words their
        kernels share between launches (the feed-forward's counts of written tiles) back to their starting values."""
        from .. import kernels
        try:
            kernels.check_status()
        except kernels.KernelError:
            torch.cuda.synchronize(self.device)
            for layer in self.model.layers:
                for part in layer.parts() if hasattr(layer, "parts") else ():
                    reset = getattr(part, "reset_after_fault", None)
                    if reset is not None:
                        reset()
            raise

    def can_take_device_tokens(self, entries: Sequence[StepEntry]) -> bool:
        """True if this batch runs as a replayed graph: single tokens that all want logits."""
        return self.use_graphs and all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries)

    # ---- decode steps as CUDA graphs ---------------------------------------------
    def _graph_step(self, entries: Sequence[StepEntry], sampling, device_tokens=None):
        import numpy as np
        lens, starts, slots = validate(entries, self.cache, self.model.vocab_size, self.max_positions,
                                       self.max_step_tokens)
        R = len(entries)
        Bp = 1
        while Bp < R:
            Bp *= 2
        mbs = tuple((max(len(e.cache.tables[g]) for e in entries) + 31) // 32 * 32
                    for g in range(len(self.cache.pools)))
        key = (Bp, mbs, sampling is not None)
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = _DecodeGraph(self, Bp, mbs, sampling is not None)
        host = g.next_host()
        h = host.numpy()
        fill(h, g.lay, entries, self.cache, lens, starts, slots, self.model.vocab_size)
        o = g.lay.off["extra"]
        if sampling is not None:
            temps, top_ks, draws = sampling
            hf = h.view(np.float32)
            hf[o:o + R] = temps
            h[o + Bp:o + Bp + R] = top_ks
            hf[o + 2 * Bp:o + 2 * Bp + R] = draws
        else:
            h[o:o + 3 * Bp] = 0
        g.upload(host)
        if device_tokens is not None:
            o = g.lay.off["tokens"]
            g.dev[o:o + R].copy_(device_tokens[:R])
            if Bp > R:      # the padding repeats entry 0 and writes to its cache slot: it must carry its token too
                g.dev[o + R:o + Bp].copy_(device_tokens[0:1].expand(Bp - R))
        g.run()
        return g.logits[:R], (g.tokens[:R] if g.tokens is not None else None)


class _NotOnHost:
    """Stands where a step's host copies of the metadata would be when the step replays as a graph."""

    def _refuse(self, *a, **k):
        raise StepError("this step replays as a CUDA graph and has no host copies of its metadata; a part whose "
                        "forward reads ctx.host_* must set needs_host_metadata = True")

    __getitem__ = __iter__ = __len__ = _refuse


class _DecodeGraph:
    """One captured decode step for a padded batch size and block-table widths."""

    def __init__(self, runner: "ModelRunner", Bp: int, mbs, with_sampling: bool):
        # no reference back to the runner: a cycle would leave the captured graph to the garbage
        # collector, which might then destroy it in the middle of another capture
        self.model = runner.model
        self.device = runner.device
        self.with_sampling = with_sampling
        self.lay = MetaLayout(Bp, Bp, Bp, mbs, extra=3 * Bp)
        # two pinned staging buffers: one may still be in flight while the next step is written
        self.hosts = [torch.empty(self.lay.total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.events = [None, None]
        self.turn = 0
        self.dev = torch.zeros(self.lay.total, dtype=torch.int32, device=runner.device)
        self.ctx = self.lay.context(self.dev, runner.cache, runner.device)
        self.ctx.all_decode = True
        self.ctx.max_portion = 1
        # nothing of a replayed step runs on the host: there are no host copies of its metadata
        self.ctx.host_cu_tokens = self.ctx.host_start_pos = self.ctx.host_state_slots = _NotOnHost()
        self.ctx.max_context = min(runner.max_positions, max(mbs) * runner.cache.page_size) if mbs else 1
        o = self.lay.off["extra"]
        self.temps = self.dev[o:o + Bp].view(torch.float32)
        self.top_ks = self.dev[o + Bp:o + 2 * Bp]
        self.draws = self.dev[o + 2 * Bp:o + 3 * Bp].view(torch.float32)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits = None
        self.tokens = None

    def next_host(self) -> torch.Tensor:
        self.turn ^= 1
        if self.events[self.turn] is not None:
            self.events[self.turn].synchronize()
        return self.hosts[self.turn]

    def upload(self, host: torch.Tensor) -> None:
        self.dev.copy_(host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[self.turn] = ev

    def _forward(self):
        from .. import kernels
        with kernels.step_stream():       # entered inside a capture too: the capturing stream is current then
            self.logits = self.model.forward(self.ctx)
            if self.with_sampling:
                self.tokens = torch.empty(self.lay.T, dtype=torch.int32, device=self.device)
                kernels.sample(self.logits, self.temps, self.top_ks, self.draws, self.tokens)

    def run(self) -> None:
        if self.graph is None:
            # the first step of this shape runs eagerly (loads every kernel), then is captured; the
            # eager run and the first replay write the same values to the same cache slots.  A state of
            # fixed size is another matter: its update is no plain write, so the eager run's is undone
            states = [st.clone() for st in self.ctx.cache.states if st is not None]
            self._forward()
            for st, saved in zip((st for st in self.ctx.cache.states if st is not None), states):
                st.copy_(saved)
            del states
            torch.cuda.synchronize(self.device)
            import gc
            from .. import kernels
            graph = torch.cuda.CUDAGraph()
            n0 = kernels.launches()
            # no garbage collection while capturing: freeing another graph or its memory in the
            # middle of a capture invalidates it
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    self._forward()
            finally:
                if gc_was_on:
                    gc.enable()
            self.own_launches = kernels.launches() - n0
            self.graph = graph
        self.graph.replay()
        from .. import kernels
        kernels.add_launches(self.own_launches)
