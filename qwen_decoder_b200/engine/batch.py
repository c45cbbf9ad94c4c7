"""A step's batch and the device metadata made from it.

The reference builds seven host vectors per step (flat tokens, positions,
token -> request, token -> cache slot, last-token indices, prefill and decode index
lists; decoder.cpp:65-163) and copies them one by one (gpu_decoder.cu:274-294),
plus changed block-table rows (gpu_decoder.cu:232-251).  Here an entry is
(request, its next tokens, the places whose logits are wanted); a decoded token is
an entry of length one.  All metadata of the step is packed into one pinned int32
buffer and copied to the device in one transfer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, RequestCache


class StepError(ValueError):
    """A batch the step function refuses (bad token id, too long, pages missing...)."""


@dataclass
class StepEntry:
    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among ``tokens`` whose logits are returned


@dataclass
class GroupView:
    """Device metadata of one paged cache group for this step."""
    block_table: torch.Tensor     # int32 [R, max_blocks]; entries of released pages are -1
    slot_map: torch.Tensor        # int32 [T]; page * page_size + offset of each token
    page_size: int
    max_blocks: int


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    device: torch.device
    tokens: torch.Tensor          # int32 [T]
    positions: torch.Tensor       # int32 [T]
    token_request: torch.Tensor   # int32 [T]; index of the token's entry in this step
    cu_tokens: torch.Tensor       # int32 [R + 1]
    start_pos: torch.Tensor       # int32 [R]
    state_slots: torch.Tensor     # int32 [R]
    logit_rows: torch.Tensor      # int32 [n_want]; flat token indices
    groups: List[GroupView]
    cache: CacheManager
    # host copies, for parts that plan on the host
    host_cu_tokens: List[int] = field(default_factory=list)
    host_start_pos: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)
    max_portion: int = 0
    max_context: int = 0
    num_wanted: int = 0


def _pad4(n: int) -> int:
    return (n + 3) & ~3


def build_context(entries: Sequence[StepEntry], cache: CacheManager, device, vocab_size: int,
                  max_positions: int) -> StepContext:
    """Validate ``entries`` and make the step's device metadata (one host-to-device copy)."""
    if not entries:
        raise StepError("a step needs at least one entry")
    R = len(entries)
    lens, starts, slots = [], [], []
    seen = set()
    for e in entries:
        n = len(e.tokens)
        rc = e.cache
        if rc.closed:
            raise StepError(f"request {rc.request_id!r} has ended")
        if id(rc) in seen:
            raise StepError(f"request {rc.request_id!r} appears twice in one step")
        seen.add(id(rc))
        if n < 1:
            raise StepError(f"request {rc.request_id!r}: an entry needs at least one token")
        if rc.num_tokens + n > max_positions:
            raise StepError(
                f"request {rc.request_id!r}: {rc.num_tokens} + {n} tokens exceed the model's "
                f"{max_positions} positions")
        for g, table in enumerate(rc.tables):
            if (rc.num_tokens + n + cache.page_size - 1) // cache.page_size > len(table):
                raise StepError(f"request {rc.request_id!r}: cache pages for its {n} new tokens are missing "
                                f"(group {g}); call ensure first")
        for w in e.want:
            if not (0 <= w < n):
                raise StepError(f"request {rc.request_id!r}: wanted place {w} is outside its {n} tokens")
        lens.append(n)
        starts.append(rc.num_tokens)
        slots.append(rc.state_slot)
    T = sum(lens)
    cu = np.zeros(R + 1, dtype=np.int64)
    np.cumsum(lens, out=cu[1:])
    tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64).reshape(-1) for e in entries])
    if tokens.min() < 0 or tokens.max() >= vocab_size:
        bad = int(tokens[(tokens < 0) | (tokens >= vocab_size)][0])
        raise StepError(f"token id {bad} is outside the vocabulary of {vocab_size}")
    token_req = np.repeat(np.arange(R, dtype=np.int64), lens)
    positions = np.arange(T, dtype=np.int64) - cu[:-1][token_req] + np.asarray(starts, dtype=np.int64)[token_req]
    want = np.concatenate([cu[i] + np.asarray(e.want, dtype=np.int64).reshape(-1)
                           for i, e in enumerate(entries)]) if any(len(e.want) for e in entries) \
        else np.zeros(0, dtype=np.int64)
    ps = cache.page_size
    n_groups = len(cache.pools)
    max_blocks = [max(1, max(len(e.cache.tables[g]) for e in entries)) for g in range(n_groups)]

    # layout of the packed buffer
    segs = {"tokens": T, "positions": T, "token_req": T, "cu": R + 1, "start": R, "slots": R, "want": len(want)}
    off, cur = {}, 0
    for k, n in segs.items():
        off[k] = cur
        cur += _pad4(n)
    goff = []
    for g in range(n_groups):
        goff.append((cur, cur + _pad4(T)))
        cur += _pad4(T) + _pad4(R * max_blocks[g])
    total = max(cur, 4)
    host = torch.empty(total, dtype=torch.int32, pin_memory=torch.device(device).type == "cuda")
    h = host.numpy()
    h[off["tokens"]:off["tokens"] + T] = tokens
    h[off["positions"]:off["positions"] + T] = positions
    h[off["token_req"]:off["token_req"] + T] = token_req
    h[off["cu"]:off["cu"] + R + 1] = cu
    h[off["start"]:off["start"] + R] = starts
    h[off["slots"]:off["slots"] + R] = slots
    h[off["want"]:off["want"] + len(want)] = want
    for g in range(n_groups):
        so, bo = goff[g]
        bt = np.full((R, max_blocks[g]), -1, dtype=np.int64)
        for i, e in enumerate(entries):
            pages = e.cache.tables[g].pages
            bt[i, :len(pages)] = pages
        page_idx = positions // ps
        phys = bt[token_req, page_idx]
        if (phys < 0).any():
            raise StepError("a token of this step would be written to a page that was given back")
        h[so:so + T] = phys * ps + positions % ps
        h[bo:bo + R * max_blocks[g]] = bt.reshape(-1)
    dev = host.to(device, non_blocking=True)

    def seg(k, n):
        return dev[off[k]:off[k] + n]

    groups = []
    for g in range(n_groups):
        so, bo = goff[g]
        groups.append(GroupView(
            block_table=dev[bo:bo + R * max_blocks[g]].view(R, max_blocks[g]),
            slot_map=dev[so:so + T], page_size=ps, max_blocks=max_blocks[g]))
    ctx = StepContext(
        num_tokens=T, num_requests=R, device=torch.device(device),
        tokens=seg("tokens", T), positions=seg("positions", T), token_request=seg("token_req", T),
        cu_tokens=seg("cu", R + 1), start_pos=seg("start", R), state_slots=seg("slots", R),
        logit_rows=seg("want", len(want)), groups=groups, cache=cache,
        host_cu_tokens=[int(c) for c in cu], host_start_pos=list(starts), host_state_slots=list(slots),
        max_portion=max(lens), max_context=max(s + n for s, n in zip(starts, lens)),
        num_wanted=len(want))
    ctx._host_buffer = host  # keep the pinned buffer alive until the copy has run
    return ctx
