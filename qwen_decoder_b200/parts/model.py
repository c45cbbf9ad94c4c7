"""A decoder put together from a ``ModelSpec``: embedding, layers run in the order
the schedule gives, final norm on the rows whose logits are wanted, output
projection to float32 logits.

Reference: forward_flat (gpu_decoder.cu:253-542).  Differences by design: the final
norm and the output projection run only on wanted rows (the reference normalises all
rows, gpu_decoder.cu:508, then gathers, :526); logits come out in float32 from the
contraction itself; the residual sum is float32 throughout.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache import CacheLayout, FixedState, PagedKV
from ..config.registry import create_part
from ..config.spec import ModelSpec, PartSpec
from ..weights.loader import TensorSource, TensorSpec
from .base import PagedCacheView, ResidualStream, StateCacheView
from .linear import Linear
# importing the part modules registers them
from . import attention as _attention, block as _block, mlp as _mlp, norm as _norm, rotary as _rotary  # noqa: F401


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size
        self.max_positions = spec.max_positions
        self.positions = {name: create_part("position", ps.name, **ps.params)
                          for name, ps in spec.positions.items()}
        self.layers = []
        for ls in spec.layers:
            mp = dict(ls.mixer.params)
            mp["prefix"] = ls.prefix + mp.get("prefix", "")
            if "position" in mp:
                pname = mp["position"]
                if pname is not None and pname not in self.positions:
                    raise ValueError(f"layer {ls.prefix!r}: unknown position encoding {pname!r}")
                mp["position"] = self.positions[pname] if pname is not None else None
            mixer = create_part("mixer", ls.mixer.name, **mp)
            fp = dict(ls.feed_forward.params)
            fp["prefix"] = ls.prefix + fp.get("prefix", "")
            ff = create_part("feed_forward", ls.feed_forward.name, **fp)
            norms = {}
            for role, ns in ls.norms.items():
                np_ = dict(ns.params)
                np_["prefix"] = ls.prefix + np_.get("prefix", "")
                norms[role] = create_part("norm", ns.name, **np_)
            self.layers.append(create_part("block", ls.block, mixer=mixer, feed_forward=ff, norms=norms))
        for i, e in enumerate(spec.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
        self.schedule = list(spec.schedule)
        fn = dict(spec.final_norm.params)
        fn["prefix"] = spec.final_norm_prefix + fn.get("prefix", "")
        self.final_norm = create_part("norm", spec.final_norm.name, **fn)
        self.lm_head = Linear(spec.hidden_size, [("lm_head", spec.vocab_size)], bias=False) \
            if spec.lm_head_tensor is None else \
            Linear(spec.hidden_size, [(spec.lm_head_tensor[:-len(".weight")], spec.vocab_size)], bias=False)
        self.embedding: Optional[torch.Tensor] = None
        self.native_prompt = None    # parts.native_prompt.NativePrompt once bound, if the parts allow it
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None

    # ---- tensors ---------------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.spec.embedding_tensor, (self.vocab_size, self.hidden_size))]
        for layer in self.layers:
            specs += layer.tensor_specs()
        specs += self.final_norm.tensor_specs()
        if self.spec.lm_head_tensor is not None:
            specs += self.lm_head.tensor_specs()
        return specs

    def ignorable_tensors(self) -> List[str]:
        """Tensors a folder may hold although this model does not use them: with tied embeddings the output
        projection reads the embedding table, and a stored output matrix is left aside."""
        return ["lm_head.weight"] if self.spec.lm_head_tensor is None else []

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.dtype, self.device = dtype, device
        self.embedding = source.get(self.spec.embedding_tensor).to(device=device, dtype=dtype).contiguous()
        for layer in self.layers:
            layer.bind(source, dtype, device)
        self.final_norm.bind(source, dtype, device)
        if self.spec.lm_head_tensor is None:
            self.lm_head.bind_tensor(self.embedding)
        else:
            self.lm_head.bind(source, dtype, device)

    def prepare(self, max_positions: int) -> None:
        """Build position tables for positions < max_positions."""
        for p in self.positions.values():
            p.prepare(min(max_positions, self.max_positions), self.device)
        self.prepared_positions = min(max_positions, self.max_positions)
        from .native_prompt import NativePrompt
        self.native_prompt = NativePrompt.try_build(self)

    def all_parts(self):
        """Every part of the model: position encodings, each layer and what it is made of, the final norm."""
        out = list(self.positions.values())
        for layer in self.layers:
            out.append(layer)
            out += list(layer.parts()) if hasattr(layer, "parts") else []
        out.append(self.final_norm)
        return out

    # ---- cache -------------------------------------------------------------
    def cache_layout(self) -> CacheLayout:
        needs = [self.layers[e.layer].mixer.cache_need() for e in self.schedule]
        return CacheLayout.from_needs(needs, [e.cache_of for e in self.schedule])

    def _cache_view(self, i: int, ctx):
        layout = ctx.cache.layout
        write = self.schedule[i].cache_of is None
        if i in layout.paged:
            g, _ = layout.paged[i]
            return PagedCacheView(kv=ctx.cache.layer_kv(i), group=ctx.groups[g], write=write)
        if i in layout.fixed:
            return StateCacheView(state=ctx.cache.layer_state(i), write=write)
        return None

    # ---- forward -------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        """Run the step's tokens through the model; float32 logits [n_wanted, vocab]."""
        x = torch.empty((ctx.num_tokens, self.hidden_size), dtype=torch.float32, device=self.device)
        kernels.embedding(x, self.embedding, ctx.tokens)
        if self.native_prompt is not None and self.native_prompt.takes(ctx):
            # the common composition, many tokens: the layers' launches come from one native loop
            h = self.native_prompt.forward(ctx, x)
            if h is None:
                return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
            return self.lm_head.forward(h, out_dtype=torch.float32)
        stream = ResidualStream(x)
        for i, e in enumerate(self.schedule):
            self.layers[e.layer].forward(stream, ctx, self._cache_view(i, ctx))
        if ctx.num_wanted == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        h = self.final_norm.forward(stream, self.dtype, rows=ctx.logit_rows)
        return self.lm_head.forward(h, out_dtype=torch.float32)


def build_model(spec: ModelSpec) -> DecoderModel:
    return DecoderModel(spec)
