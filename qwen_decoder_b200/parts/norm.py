"""RMSNorm: out = x / sqrt(mean(x^2) + eps) * w, statistics in float32, weight as ``w``
(not ``1 + w``), as the reference's rmsnorm_kernel (gpu_kernels.cu:32-67) and its CPU
form (cpu_decoder.cpp:48-53) — with eps a parameter where the reference has the
literal 1e-6 (gpu_kernels.cu:63).  The kernel also adds the residual branch that is
still pending on the stream, which the reference does in a separate residual_kernel
(gpu_kernels.cu:136-146).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Norm, ResidualStream


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, size: int, eps: float, prefix: str = ""):
        self.size = size
        self.eps = float(eps)
        self.prefix = prefix
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(f"{self.prefix}weight", (self.size,), init="around_one")]

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        # norm scales are used in float32 whatever they are stored in
        self.weight = source.get(f"{self.prefix}weight").to(device=device, dtype=torch.float32).contiguous()

    def native_params(self) -> Optional[dict]:
        return {"kind": "rmsnorm", "weight": self.weight, "eps": self.eps, "size": self.size}

    def forward(self, stream: ResidualStream, out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = stream.x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=stream.x.device)
        kernels.add_rmsnorm(stream.x, stream.delta, self.weight, out, self.eps, rows=rows,
                            write_back=rows is None)
        if rows is None:
            stream.delta = None
        return out
