"""Which kernel a contraction runs on.

float32: always the float32 FMA kernel (``csrc/gemm_generic.cu``); no TF32 anywhere.
bfloat16: ``mode`` chooses.
  * ``auto``    few tokens (<= 64): the hand-written weight-streaming tensor-core kernel
                (``csrc/gemm_skinny.cu``); more tokens: cuBLAS for products large enough to
                matter, else the generic kernel;
  * ``generic`` always the generic kernel (any size);
  * ``cublas``  the library product through torch, as the reference calls cublasHgemm
                (gpu_kernels.cu:431-436), for every bfloat16 product.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import kernels

mode = os.environ.get("QD_BF16_GEMM", "auto")

# bookkeeping for benchmarks: how many launches of our own kernels / library products ran
counters = {"own": 0, "library": 0}


_bias_copies = {}     # (address of the float32 bias, dtype) -> (the bias itself, its copy in that dtype)


def _bias_as(bias: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The library product adds a bias of the output's dtype: convert each bias once, not every call."""
    key = (bias.data_ptr(), dtype)
    hit = _bias_copies.get(key)
    if hit is None or hit[0] is not bias:
        hit = _bias_copies[key] = (bias, bias.to(dtype))
    return hit[1]


def _cublas(x, w, bias, out):
    if out.dtype == torch.float32:
        y = torch.mm(x, w.t(), out_dtype=torch.float32)
        if bias is not None:
            y += bias
        out.copy_(y)
    elif bias is not None:
        torch.addmm(_bias_as(bias, out.dtype), x, w.t(), out=out)
    else:
        torch.mm(x, w.t(), out=out)
    counters["library"] += 1


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[T, N] = x[T, K] @ w[N, K]^T (+ bias[N] float32)."""
    if not x.is_cuda:
        raise kernels.KernelError("contractions run on a CUDA device only (there is no CPU path)")
    if x.dtype == torch.float32 or mode == "generic":
        kernels.gemm_generic(x, w, bias, out)
        counters["own"] += 1
        return
    if mode == "cublas":
        _cublas(x, w, bias, out)
        return
    T, K = x.shape
    N = w.shape[0]
    if kernels.skinny_supported(x, w) and out.stride(1) == 1:
        kernels.gemm_skinny(x, w, bias, out)
        counters["own"] += 1
        return
    if K % 8 == 0 and N % 8 == 0 and N * K >= 256 * 256:
        _cublas(x, w, bias, out)
    else:
        kernels.gemm_generic(x, w, bias, out)
        counters["own"] += 1


# A library product of few tokens with a long K and few output features (the down projection of 17 to 256 tokens)
# fills the GPU with too few CTAs.  Given as a batch over four shares of K that leaves float32 partial sums it is
# faster: decode steps at the 3B sizes 3.11 -> 2.92 ms at batch 64 and 2.60 -> 2.44 at batch 32 (2 and 8 shares:
# 2.95), at the 7B sizes 3.81 -> 3.69 at batch 32, nothing with 5,120 output features; the product alone on cold
# weights 17.5 -> 12.0 us at 128 tokens and 18.8 -> 13.5 at 256.
# It is OFF (``library_split_k = 0``; 4 turns it on).  With it on, tests at the 3B and 7B sizes saw, in about one
# run of ten, one row tile of a LATER prompt step's logits wrong (a 268- or 291-token portion, always the rows from
# 128 on), also when that step's own products were plain ones and with the batched product's reader and writer
# ordered by plain launches; five runs with it off showed none, as did all runs before it existed.  The cause was
# not found (what the library's kernels keep between calls cannot be seen from here), so the plain product stands.
library_split_k = 0
LIBRARY_SPLIT_MAX_FEATURES = 4096
LIBRARY_SPLIT_MAX_TOKENS = 256


def library_shares(T: int, N: int, K: int) -> int:
    """Shares of K for ``linear_partial_library`` and for the native prompt loop's down projection, or 0 where
    the plain library product stands."""
    if (mode != "auto" or library_split_k < 2 or not (16 < T <= LIBRARY_SPLIT_MAX_TOKENS)
            or N > LIBRARY_SPLIT_MAX_FEATURES or K < 2 * N or K < 4096):
        return 0
    s = library_split_k
    return s if K % (8 * s) == 0 else 0


def linear_partial_library(x: torch.Tensor, w: torch.Tensor, shares: int) -> torch.Tensor:
    """float32 partial sums [shares, T, N] of x @ w^T over equal shares of K, as one batched library product on
    strided views (nothing is copied)."""
    T, K = x.shape
    N = w.shape[0]
    kc = K // shares
    xs = x.view(T, shares, kc).transpose(0, 1)              # [S, T, kc]
    ws = w.view(N, shares, kc).permute(1, 2, 0)             # [S, kc, N]
    counters["library"] += 1
    part = torch.bmm(xs, ws, out_dtype=torch.float32)
    kernels.elementwise_plain_next()          # whoever adds these sums up waits for the whole batched product
    return part


def use_skinny(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the few-token kernel (and its fused epilogues) takes this product."""
    return mode == "auto" and x.is_cuda and kernels.skinny_supported(x, w)
