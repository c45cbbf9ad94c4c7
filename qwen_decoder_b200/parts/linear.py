"""A contraction y = x W^T (+ b) with weights row-major [out_features, in_features]
(the reference's layout, common.h:33-43; y[t,o] = sum_i x[t,i] W[o,i],
cpu_decoder.cpp:55-62).  Several named tensors may be stacked along the output
dimension at bind time (q, k and v into one product; gate and up into one), which
the reference runs as separate cublasHgemm calls (gpu_decoder.cu:334-336, 457-466).

Which kernel runs is decided here by dtype and size: the float32 path always takes
the float32 FMA kernel; the bfloat16 path takes the tensor-core kernel where its
sizes allow and the generic kernel otherwise.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .. import kernels
from ..weights.loader import TensorSource, TensorSpec
from . import matmul_backend


class Linear:
    def __init__(self, in_features: int, pieces: Sequence[Tuple[str, int]], bias: bool):
        """``pieces``: (weight-name stem, out_features) stacked in order; tensor names are
        ``<stem>.weight`` and, with ``bias``, ``<stem>.bias``."""
        self.in_features = in_features
        self.pieces = list(pieces)
        self.out_features = sum(n for _, n in pieces)
        self.has_bias = bias
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = []
        for stem, n in self.pieces:
            specs.append(TensorSpec(f"{stem}.weight", (n, self.in_features)))
            if self.has_bias:
                specs.append(TensorSpec(f"{stem}.bias", (n,)))
        return specs

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        ws = [source.get(f"{stem}.weight").to(device=device, dtype=dtype) for stem, _ in self.pieces]
        self.weight = (torch.cat(ws, dim=0) if len(ws) > 1 else ws[0]).contiguous()
        if self.has_bias:
            bs = [source.get(f"{stem}.bias").to(device=device, dtype=torch.float32) for stem, _ in self.pieces]
            self.bias = (torch.cat(bs, dim=0) if len(bs) > 1 else bs[0]).contiguous()

    def bind_tensor(self, weight: torch.Tensor) -> None:
        """Use an already prepared weight (a tied output projection shares the embedding table)."""
        self.weight = weight

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.dtype, device=x.device)
        matmul_backend.linear(x, self.weight, self.bias, out)
        return out

    def forward_partial(self, x: torch.Tensor) -> torch.Tensor:
        """The product as something a residual stream can take: [T, N] in x's dtype, or -- from the
        few-token kernel -- float32 partial sums [n_parts, T, N] (bias not added) that the next
        norm's kernel adds up."""
        if self.bias is None and matmul_backend.use_skinny(x, self.weight):
            matmul_backend.counters["own"] += 1
            return kernels.gemm_skinny_partial(x, self.weight, kernels.skinny_splits(self.out_features, self.in_features, x.shape[0]))
        if self.bias is None and x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous():
            shares = matmul_backend.library_shares(x.shape[0], self.out_features, self.in_features)
            if shares:
                return matmul_backend.linear_partial_library(x, self.weight, shares)
        return self.forward(x)
