"""The pre-norm residual block: x += mixer(norm(x)); x += feed_forward(norm(x))
(gpu_decoder.cu:321-497: norm, attention, residual, norm, feed-forward, residual).
A branch's output is left pending on the stream and added by the next norm's kernel.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Block, FeedForward, Mixer, Norm, ResidualStream


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    norm_roles = ("input", "post_mixer")

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm]):
        missing = [r for r in self.norm_roles if r not in norms]
        if missing:
            raise ValueError(f"pre_norm block needs norms {self.norm_roles}, missing {missing}")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.input_norm = norms["input"]
        self.post_mixer_norm = norms["post_mixer"]

    def parts(self):
        return [self.input_norm, self.mixer, self.post_mixer_norm, self.feed_forward]

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self.parts() for s in p.tensor_specs()]

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.dtype = dtype
        for p in self.parts():
            p.bind(source, dtype, device)

    def native_params(self):
        if type(self) is not PreNormBlock:
            return None          # a subclass may run its parts in another order: it answers for itself
        n1, mx = self.input_norm.native_params(), self.mixer.native_params()
        n2, ff = self.post_mixer_norm.native_params(), self.feed_forward.native_params()
        if None in (n1, mx, n2, ff) or not all(k in mx for k in ("wqkv", "wo", "H", "G", "d")) \
                or not all(k in ff for k in ("wgu", "wd", "F")) or "weight" not in n1 or "weight" not in n2:
            return None
        if not (n1["size"] == n2["size"] == mx["D"] == ff["D"]):
            return None
        out = dict(mx)
        # what runs in which order: native code that restates one composition takes that one only
        out["composition"] = "/".join(["pre_norm", str(mx.get("kind")), str(ff.get("kind")), str(n1.get("kind")),
                                       str(n2.get("kind"))])
        out.update(F=ff["F"], wgu=ff["wgu"], wd=ff["wd"], norm1_w=n1["weight"], eps1=n1["eps"],
                   norm2_w=n2["weight"], eps2=n2["eps"])
        return out

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        h = self.input_norm.forward(stream, self.dtype)
        stream.push(self.mixer.forward(h, ctx, cache))
        h = self.post_mixer_norm.forward(stream, self.dtype)
        stream.push(self.feed_forward.forward(h, ctx))
