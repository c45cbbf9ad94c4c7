"""Sampling above the step function: greedy, temperature, top-k, on the device.

The distribution is the reference's (common.cpp:576-629; see ``csrc/sampling.cu``).
The reference draws from one std::mt19937 shared by all requests in batch order
(decoder.cpp:201-202, gpu_main.cu:45), so its output depends on the batch a request is
in.  Here the uniform draw of a request's i-th output token is a counter-based hash of
(seed, request key, i): the same request gives the same tokens whatever runs beside it,
and again after a preemption.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import kernels

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_draw(seed: int, key: int, index: int) -> float:
    """A float32 in [0, 1) that depends only on (seed, key, index)."""
    h = _splitmix64(_splitmix64(_splitmix64(seed & _MASK) ^ (key & _MASK)) ^ (index & _MASK))
    return float(np.float32((h >> 40) * (1.0 / (1 << 24))))


class Sampler:
    """Samples one token per logits row on the device; returns a device int32 tensor."""

    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], top_ks: Sequence[int],
               draws: Sequence[float]) -> torch.Tensor:
        R = logits.shape[0]
        host = torch.empty((3, max(R, 1)), dtype=torch.float32, pin_memory=True)
        host[0, :R] = torch.tensor(list(temperatures), dtype=torch.float32)
        host[1, :R] = torch.tensor(list(draws), dtype=torch.float32)
        host[2, :R] = torch.tensor(list(top_ks), dtype=torch.int32).view(torch.float32)
        dev = host.to(self.device, non_blocking=True)
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        kernels.sample(logits, dev[0, :R], dev[2, :R].view(torch.int32), dev[1, :R], out)
        return out

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        R = logits.shape[0]
        zeros = torch.zeros(R, dtype=torch.float32, device=self.device)
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        kernels.sample(logits, zeros, zeros.view(torch.int32), zeros, out)
        return out
