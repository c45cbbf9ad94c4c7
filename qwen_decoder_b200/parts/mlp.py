"""SwiGLU feed-forward: h = silu(x W1^T) * (x W3^T); delta = h W2^T, no biases
(gpu_decoder.cu:457-497, swiglu_kernel gpu_kernels.cu:149-160, cpu_decoder.cpp:204-212;
W1 = gate_proj, W3 = up_proj, W2 = down_proj).  Gate and up are one stacked product.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import FeedForward
from . import matmul_backend
from .linear import Linear


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "mlp."):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate_up = Linear(hidden_size, [(f"{prefix}gate_proj", intermediate_size),
                                            (f"{prefix}up_proj", intermediate_size)], bias=False)
        self.down = Linear(intermediate_size, [(f"{prefix}down_proj", hidden_size)], bias=False)
        self._barrier = None

    def tensor_specs(self) -> List[TensorSpec]:
        return self.gate_up.tensor_specs() + self.down.tensor_specs()

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.gate_up.bind(source, dtype, device)
        self.down.bind(source, dtype, device)

    def native_params(self):
        return {"kind": "swiglu", "D": self.hidden_size, "F": self.intermediate_size, "wgu": self.gate_up.weight,
                "wd": self.down.weight}

    def reset_after_fault(self) -> None:
        """A launch whose wait for the other CTAs ran out may have left tiles counted: start from zero again."""
        if self._barrier is not None:
            self._barrier.zero_()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        if matmul_backend.mode == "auto" and kernels.ffn_stream_supported(x, self.gate_up.weight, self.down.weight):
            matmul_backend.counters["own"] += 1
            if self._barrier is None:       # this layer's own synchronisation words (zero once; each launch leaves them zero)
                self._barrier = torch.zeros(kernels.FFN_SYNC_WORDS, dtype=torch.int32, device=x.device)
            return kernels.ffn_stream(x, self.gate_up.weight, self.down.weight, self._barrier)   # one launch
        h = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        if matmul_backend.use_skinny(x, self.gate_up.weight):
            shares = kernels.swiglu_shares(x.shape[0], self.hidden_size, 2 * self.intermediate_size)
            if shares and self.intermediate_size % 4 == 0:
                # where the streamer keeps the tokens resident only for a share of K: partial sums, then SwiGLU
                kernels.swiglu_partial(kernels.gemm_skinny_partial(x, self.gate_up.weight, shares), h)
            else:
                kernels.gemm_skinny_swiglu(x, self.gate_up.weight, h)       # gate, up and SwiGLU in one kernel
            matmul_backend.counters["own"] += 1
        else:
            kernels.swiglu(self.gate_up.forward(x), h)
        return self.down.forward_partial(h)
