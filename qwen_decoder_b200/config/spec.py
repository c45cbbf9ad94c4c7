"""A model written down as data: which parts each layer is made of, with which
sizes and constants, and in which order the layers run.

Nothing here knows an architecture.  An architecture is a function from its typed
configuration to a ``ModelSpec`` (see ``config.qwen2`` for the one this engine ships).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """A registered part by name, with its sizes and constants."""
    name: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (block) of a mixer, a feed-forward and norms.

    ``prefix`` is the weight-name prefix of the layer (``model.layers.3.``).
    ``norms`` maps the block's norm roles to part specs (for the pre-norm block:
    ``input`` and ``post_mixer``).
    """
    prefix: str
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named more than once).
    ``cache_of`` names the schedule entry whose cache this run uses: ``None`` means
    its own (the run writes what its mixer caches); an integer ``j < i`` means "read
    what entry ``j`` cached", without writing.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_tensor: str
    positions: Dict[str, PartSpec]          # position encodings, shared by name
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    final_norm_prefix: str
    lm_head_tensor: Optional[str]           # None: tied to the embedding
