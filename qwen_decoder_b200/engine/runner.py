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
from .batch import StepEntry, StepError, build_context

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
                 max_requests: int = 64, max_positions: Optional[int] = None):
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
                                  device=self.device)
        self.steps = 0
        self.tokens_run = 0

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
    def open(self, request_id) -> RequestCache:
        return self.cache.open(request_id)

    def close(self, rc: RequestCache) -> None:
        self.cache.close(rc)

    # ---- the step ------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], ensure_pages: bool = True) -> torch.Tensor:
        """Run one batch; returns float32 logits [wanted places in entry order, vocab] on the device.

        With ``ensure_pages`` the pages the new tokens need are taken first (``OutOfPages`` if the
        pool cannot give them; nothing is taken then).  Afterwards each request's cached length has
        grown by its tokens."""
        if ensure_pages:
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
        ctx = build_context(entries, self.cache, self.device, self.model.vocab_size, self.max_positions)
        logits = self.model.forward(ctx)
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens))
        self.steps += 1
        self.tokens_run += ctx.num_tokens
        return logits
