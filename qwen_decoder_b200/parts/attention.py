"""Grouped-query attention over the paged cache.

As the reference computes it: q, k, v = x Wq^T + bq, x Wk^T + bk, x Wv^T + bv
(gpu_decoder.cu:334-349); head h of q is columns h*d .. h*d+d-1 and reads kv head
h / (H / G) (gpu_kernels.cu:222,232); q and k are rotated by position, then k and v are
written to the token's cache slot (gpu_kernels.cu:82-133); a query at position pos
attends keys 0..pos with scores (q.k) / sqrt(d), softmax, weighted sum of v
(gpu_kernels.cu:223-311; cpu_decoder.cpp:166-193); the result goes through Wo with no
bias (gpu_decoder.cu:423).  Prompt portions and decoded tokens run through the same
kernels: a portion's keys are in the pages before its queries read them.
``window`` = w limits a query to the last w keys (the reference has no window).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import kernels
from ..cache import PagedKV
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Mixer, PagedCacheView
from . import matmul_backend
from .linear import Linear


@register_part("mixer", "gq_attention")
class GQAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool = True, out_bias: bool = False, position=None,
                 window: Optional[int] = None, prefix: str = "self_attn.", scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_kv_heads ({num_kv_heads}) must divide num_heads ({num_heads})")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.window = window
        self.position = position        # a PositionEncoding part (Rotary) or None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.qkv = Linear(hidden_size, [(f"{prefix}q_proj", num_heads * head_dim),
                                        (f"{prefix}k_proj", num_kv_heads * head_dim),
                                        (f"{prefix}v_proj", num_kv_heads * head_dim)], bias=qkv_bias)
        self.out = Linear(num_heads * head_dim, [(f"{prefix}o_proj", hidden_size)], bias=out_bias)

    def cache_need(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> List[TensorSpec]:
        return self.qkv.tensor_specs() + self.out.tensor_specs()

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.qkv.bind(source, dtype, device)
        self.out.bind(source, dtype, device)

    def native_params(self):
        from .rotary import Rotary
        pos = self.position
        if self.out.bias is not None or not (pos is None or type(pos) is Rotary):
            return None
        return {"kind": "gq_attention", "D": self.hidden_size, "H": self.num_heads, "G": self.num_kv_heads, "d": self.head_dim,
                "window": self.window, "scale": self.scale, "position": pos,
                "rotary_dim": pos.rotary_dim if pos is not None else 0,
                "pairing": pos.pairing_code if pos is not None else 0,
                "wqkv": self.qkv.weight, "bqkv": self.qkv.bias, "wo": self.out.weight}

    def forward(self, x: torch.Tensor, ctx, cache: PagedCacheView) -> torch.Tensor:
        H, G, d = self.num_heads, self.num_kv_heads, self.head_dim
        pos = self.position
        rope = (pos.rotary_dim if pos is not None else 0, pos.pairing_code if pos is not None else 0,
                pos.cos if pos is not None else None, pos.sin if pos is not None else None)
        if matmul_backend.use_skinny(x, self.qkv.weight):
            # few tokens: the product leaves float32 partial sums; bias, rotation and cache write take them
            part = kernels.gemm_skinny_partial(x, self.qkv.weight,
                                               kernels.skinny_splits(self.qkv.out_features, self.hidden_size, x.shape[0]))
            matmul_backend.counters["own"] += 1
            ps, window = cache.group.page_size, self.window or 0
            if ctx.all_decode and _DECODE_ROPE and kernels.decode_rope_supported(x.dtype, H, G, d, ps):
                # ... and so does attention itself: one kernel from the partial sums to the attention output
                attn = torch.empty((x.shape[0], H * d), dtype=x.dtype, device=x.device)
                kernels.decode_attention_rope(
                    part, self.qkv.bias, attn, cache.kv, cache.group.block_table, ctx.token_request, ctx.positions,
                    cache.group.slot_map, H, G, d, ps, self.scale, window,
                    decode_rope_splits(ctx.num_tokens * G, min(ctx.max_context, window or ctx.max_context)),
                    cache.write, *rope)
                return self.out.forward_partial(attn)
            qkv = torch.empty((x.shape[0], H * d), dtype=x.dtype, device=x.device)       # q only
            kernels.rope_kv_write_partial(part, self.qkv.bias, qkv, H, G, d, *rope, ctx.positions, cache.kv,
                                          cache.group.slot_map, cache.group.page_size, cache.write)
        else:
            qkv = self.qkv.forward(x)
            kernels.rope_kv_write(qkv, H, G, d, *rope, ctx.positions, cache.kv, cache.group.slot_map,
                                  cache.group.page_size, cache.write)
        attn = torch.empty((x.shape[0], H * d), dtype=x.dtype, device=x.device)
        ps, window = cache.group.page_size, self.window or 0
        if ctx.all_decode and kernels.flash_decode_supported(x.dtype, H, G, d, ps):
            kernels.decode_attention(
                qkv, qkv.stride(0), attn, cache.kv, cache.group.block_table, ctx.token_request,
                ctx.positions, ctx.num_tokens, H, G, d, ps, self.scale, window,
                decode_splits(ctx.num_tokens * G, min(ctx.max_context, window or ctx.max_context)))
        elif kernels.flash_prefill_supported(x.dtype, H, G, d, ps) or \
                (_PREFILL_TC5 and kernels.prefill_tc5_supported(x.dtype, H, G, d, ps)):
            # a mixed step: its single tokens (first in the batch) go to the decode kernel, which shares
            # a request's keys among CTAs; a prompt kernel would walk them with one CTA per request
            nd = getattr(ctx, "num_decode", 0)
            if nd and not kernels.flash_decode_supported(x.dtype, H, G, d, ps):
                nd = 0
            if nd:
                kernels.decode_attention(
                    qkv, qkv.stride(0), attn[:nd], cache.kv, cache.group.block_table, ctx.token_request[:nd],
                    ctx.positions[:nd], nd, H, G, d, ps, self.scale, window,
                    decode_splits(nd * G, min(ctx.decode_max_context, window or ctx.decode_max_context)))
            fn = kernels.prefill_attention_tc5 \
                if _PREFILL_TC5 and kernels.prefill_tc5_supported(x.dtype, H, G, d, ps) else kernels.prefill_attention
            fn(qkv, qkv.stride(0), attn, cache.kv, cache.group.block_table[nd:], ctx.cu_tokens[nd:],
               ctx.start_pos[nd:], ctx.num_requests - nd, ctx.num_tokens - nd, H, G, d, ps, self.scale, window)
        else:
            kernels.paged_attention_generic(
                qkv, qkv.stride(0), attn, cache.kv, cache.group.block_table, ctx.token_request,
                ctx.positions, ctx.num_tokens, H, G, d, ps, self.scale, window)
        return self.out.forward_partial(attn)


import os as _os
_DECODE_ROPE = _os.environ.get("QD_DECODE_ROPE", "1") != "0"
_PREFILL_TC5 = _os.environ.get("QD_PREFILL_TC5", "1") != "0"      # prompt portions on tcgen05 where its sizes allow


def decode_rope_splits(ctas_without_split: int, max_keys: int) -> int:
    """CTAs (of 8 warps) per (request, kv head) in the kernel that also rotates and writes the cache: one
    CTA for each multiprocessor (two were slower in whole decode steps at batch 4 and 8, equal at 1 and 2),
    never more than that, and none with fewer than eight 16-key chunks, one per warp."""
    by_fill = max(1, kernels.sm_count() // max(1, ctas_without_split))      # never a second wave
    by_work = max(1, (max_keys + 127) // 128)
    return max(1, min(by_fill, by_work, 64))


def decode_splits(ctas_without_split: int, max_keys: int, target_ctas: Optional[int] = None) -> int:
    """How many CTAs share one (request, kv head) in decode attention: enough for one CTA on each of
    the multiprocessors (more splits cost more in the combine than they gain: measured in whole decode steps at
    batch 1, 8 and 64), but no CTA with fewer than four 16-key chunks."""
    if target_ctas is None:
        target_ctas = kernels.sm_count()
    by_fill = max(1, -(-target_ctas // max(1, ctas_without_split)))
    by_work = max(1, (max_keys + 63) // 64)
    return max(1, min(by_fill, by_work, 64))
