"""Rotary position encoding.

The reference computes, per element and per layer, theta_p = 1 / base^(2p/d), the
angle theta_p * pos, and rotates the adjacent pair (2p, 2p+1) of every q and k head
(gpu_kernels.cu:82-112; cpu_decoder.cpp:135-157).  Here the cosines and sines are a
float32 table [positions, rotary_dim / 2], made once from angles taken in float64,
and the rotation is fused with the cache write (``csrc/elementwise.cu``).
``pairing`` = "adjacent" is the reference's; "half" pairs (p, p + rotary_dim / 2).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.registry import register_part
from .base import PositionEncoding

PAIRING_CODES = {"adjacent": 0, "half": 1}


@register_part("position", "rotary")
class Rotary(PositionEncoding):
    def __init__(self, head_dim: int, rotary_dim: int, base: float, pairing: str = "adjacent"):
        if pairing not in PAIRING_CODES:
            raise ValueError(f"rotary pairing must be one of {sorted(PAIRING_CODES)}, got {pairing!r}")
        if rotary_dim % 2 or not (0 < rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim ({rotary_dim}) must be even and at most head_dim ({head_dim})")
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim
        self.base = float(base)
        self.pairing = pairing
        self.pairing_code = PAIRING_CODES[pairing]
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def prepare(self, max_positions: int, device: torch.device) -> None:
        p = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        inv_freq = 1.0 / torch.pow(torch.tensor(self.base, dtype=torch.float64), 2.0 * p / self.rotary_dim)
        angle = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.cos = angle.cos().to(torch.float32).to(device).contiguous()
        self.sin = angle.sin().to(torch.float32).to(device).contiguous()
