"""Interfaces of the parts a layer is put together from.

A part has its sizes and constants as constructor parameters, declares the tensors
it needs by full name (``tensor_specs``), takes them in ``bind`` and computes in
``forward``.  No part knows which model it is in: a mixer sees the step's context
and a view of its own cache, nothing else.

Kinds of parts (each has a registry, see ``config.registry``):

* ``norm``          ``forward(stream, out_dtype, rows=None) -> normed [n, D]``
* ``position``      ``prepare(max_positions, device)``; a mixer asks it to ``rotate``
* ``mixer``         ``cache_need()``; ``forward(x [T, D], ctx, cache) -> delta [T, D]``
* ``feed_forward``  ``forward(x [T, D], ctx) -> delta [T, D]``
* ``block``         ``forward(stream, ctx, cache)``: the arrangement of the above
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSource, TensorSpec


class Part:
    """Base of every part: tensors by name, bound once, then ``forward``."""

    # True if ``forward`` reads the host copies of the step's metadata (``ctx.host_cu_tokens``,
    # ``ctx.host_start_pos``, ``ctx.host_state_slots``): a loop over requests in Python.  A step that is
    # replayed as a CUDA graph has no such copies (nothing of it runs on the host), so a model with such
    # a part runs every step eagerly.  Parts that work from the device tensors alone leave it False.
    needs_host_metadata = False

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        pass

    def native_params(self) -> Optional[dict]:
        """The part's tensors and constants, if native code may stand in for its ``forward``: the native
        prompt loop (``parts/native_prompt.py``) runs a model only when every part of it answers.  None,
        the default, keeps the part's own path."""
        return None


class ResidualStream:
    """The residual sum of a step: ``x`` float32 [T, D], and a branch output ``delta`` that has
    not been added yet (the next norm adds it in the same kernel that normalises)."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.delta: Optional[torch.Tensor] = None

    def push(self, delta: torch.Tensor) -> None:
        """Hand over a branch output; a delta still pending is added first."""
        self.flush()
        self.delta = delta

    def flush(self) -> None:
        if self.delta is not None:
            kernels.residual_add(self.x, self.delta)
            self.delta = None


@dataclass
class PagedCacheView:
    """A mixer's view of its paged cache in this step."""
    kv: torch.Tensor            # [pages, 2, kv heads, page_size, head_dim]
    group: object               # engine.batch.GroupView
    write: bool                 # False when this run reads another run's cache


@dataclass
class StateCacheView:
    """A mixer's view of its fixed-size per-request state in this step."""
    state: torch.Tensor         # [slots, *shape]
    write: bool


class Mixer(Part):
    def cache_need(self):
        """``PagedKV``, ``FixedState`` or None."""
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, stream: ResidualStream, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, max_positions: int, device: torch.device) -> None:
        pass


class Block(Part):
    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        raise NotImplementedError
