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

import os

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
    all_decode: bool = False      # every entry is one token (the kernels may take a decode path)
    # In a step that mixes single tokens with longer portions the single tokens come first in the flat
    # batch (entries are reordered inside the step; logits keep the caller's order): requests and tokens
    # 0 .. num_decode-1 are those, and a mixer may give them to its decode kernel.  0 when not mixed.
    num_decode: int = 0
    decode_max_context: int = 0   # most keys any of them reads


# single tokens first in a mixed step, for the mixers' decode kernels
_SPLIT_MIXED = True


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class MetaLayout:
    """Where each array lies in the packed int32 buffer, for given (padded) sizes."""

    def __init__(self, T: int, R: int, n_want: int, max_blocks: Sequence[int], extra: int = 0):
        self.T, self.R, self.n_want, self.max_blocks = T, R, n_want, list(max_blocks)
        segs = {"tokens": T, "positions": T, "token_req": T, "cu": R + 1, "start": R, "slots": R,
                "want": n_want, "extra": extra}
        self.off, cur = {}, 0
        for k, n in segs.items():
            self.off[k] = cur
            cur += _pad4(n)
        self.goff = []
        for mb in self.max_blocks:
            self.goff.append((cur, cur + _pad4(T)))
            cur += _pad4(T) + _pad4(R * mb)
        self.total = max(cur, 4)

    def context(self, dev: torch.Tensor, cache: CacheManager, device, n_want: Optional[int] = None) -> StepContext:
        """Views into the device copy ``dev`` of the packed buffer."""
        T, R = self.T, self.R
        nw = self.n_want if n_want is None else n_want
        seg = lambda k, n: dev[self.off[k]:self.off[k] + n]
        groups = []
        for g, mb in enumerate(self.max_blocks):
            so, bo = self.goff[g]
            groups.append(GroupView(block_table=dev[bo:bo + R * mb].view(R, mb), slot_map=dev[so:so + T],
                                    page_size=cache.page_size, max_blocks=mb))
        return StepContext(
            num_tokens=T, num_requests=R, device=torch.device(device),
            tokens=seg("tokens", T), positions=seg("positions", T), token_request=seg("token_req", T),
            cu_tokens=seg("cu", R + 1), start_pos=seg("start", R), state_slots=seg("slots", R),
            logit_rows=seg("want", nw), groups=groups, cache=cache, num_wanted=nw)


def validate(entries: Sequence[StepEntry], cache: CacheManager, vocab_size: int, max_positions: int,
             max_step_tokens: Optional[int] = None):
    """Check a batch; returns (lens, starts, slots)."""
    if not entries:
        raise StepError("a step needs at least one entry")
    if max_step_tokens is not None:
        total = sum(len(e.tokens) for e in entries)
        if total > max_step_tokens:
            raise StepError(f"the step holds {total} tokens, more than max_step_tokens = {max_step_tokens}")
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
    return lens, starts, slots


def fill(h: np.ndarray, lay: MetaLayout, entries: Sequence[StepEntry], cache: CacheManager, lens, starts,
         slots, vocab_size: int, want_order: Optional[Sequence[int]] = None):
    """Write the step's arrays into the host buffer ``h`` (int32) at ``lay``'s places.  When ``lay``
    is larger than the batch (a padded decode batch), the padding repeats entry 0's token, position and
    block table, and writes to the cache's scratch page and scratch state slot.  ``want_order``: the
    order of the entries in which their wanted rows are listed (default: as given)."""
    R = len(entries)
    T = sum(lens)
    cu = np.zeros(R + 1, dtype=np.int64)
    np.cumsum(lens, out=cu[1:])
    if T == R:
        tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=R)
    else:
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64).reshape(-1) for e in entries])
    if tokens.min() < 0 or tokens.max() >= vocab_size:
        bad = int(tokens[(tokens < 0) | (tokens >= vocab_size)][0])
        raise StepError(f"token id {bad} is outside the vocabulary of {vocab_size}")
    starts_a = np.asarray(starts, dtype=np.int64)
    if T == R:
        token_req = np.arange(R, dtype=np.int64)
        positions = starts_a
    else:
        token_req = np.repeat(np.arange(R, dtype=np.int64), lens)
        positions = np.arange(T, dtype=np.int64) - cu[:-1][token_req] + starts_a[token_req]
    want = [cu[i] + np.asarray(entries[i].want, dtype=np.int64).reshape(-1)
            for i in (range(R) if want_order is None else want_order) if len(entries[i].want)]
    want = np.concatenate(want) if want else np.zeros(0, dtype=np.int64)
    padded = lay.T != T or lay.R != R
    if padded and not (T == R and lay.T == lay.R and len(want) == R):
        raise StepError("only a batch of single tokens that all want logits can be padded")

    def put(key, arr, n_real, n_pad):
        o = lay.off[key]
        h[o:o + n_real] = arr
        if n_pad > n_real:
            h[o + n_real:o + n_pad] = arr[0]

    put("tokens", tokens, T, lay.T)
    put("positions", positions, T, lay.T)
    o = lay.off["token_req"]
    h[o:o + lay.T] = np.arange(lay.T) if padded else token_req
    o = lay.off["cu"]
    h[o:o + lay.R + 1] = np.arange(lay.R + 1) if padded else cu
    put("start", starts_a, R, lay.R)
    put("slots", np.asarray(slots, dtype=np.int64), R, lay.R)
    if lay.R > R:
        # padding rows repeat entry 0 where that is harmless (the same K/V written twice); a state of fixed
        # size would be updated twice, so they get the slot that belongs to no request
        o = lay.off["slots"]
        h[o + R:o + lay.R] = cache.scratch_slot
    o = lay.off["want"]
    h[o:o + lay.n_want] = np.arange(lay.n_want) if padded else want
    ps = cache.page_size
    for g, mb in enumerate(lay.max_blocks):
        so, bo = lay.goff[g]
        bt = np.full((lay.R, mb), -1, dtype=np.int64)
        for i, e in enumerate(entries):
            pages = e.cache.tables[g].pages
            bt[i, :len(pages)] = pages
        if lay.R > R:
            bt[R:] = bt[0]
        phys = bt[token_req, positions // ps]
        if (phys < 0).any():
            raise StepError("a token of this step would be written to a page that was given back")
        put_arr = phys * ps + positions % ps
        h[so:so + T] = put_arr
        if lay.T > T:
            # padding rows read what entry 0 reads, but what they compute may differ from entry 0's (a state of
            # their own): their keys and values go to the page that belongs to no request
            h[so + T:so + lay.T] = cache.scratch_page * ps
        h[bo:bo + lay.R * mb] = bt.reshape(-1)
    return cu, want


def build_context(entries: Sequence[StepEntry], cache: CacheManager, device, vocab_size: int,
                  max_positions: int, max_step_tokens: Optional[int] = None) -> StepContext:
    """Validate ``entries`` and make the step's device metadata (one host-to-device copy)."""
    lens, starts, slots = validate(entries, cache, vocab_size, max_positions, max_step_tokens)
    R, T = len(entries), sum(lens)
    # single tokens first when the step mixes them with longer portions (stable otherwise)
    n_single = sum(1 for n in lens if n == 1)
    want_order = None
    if 0 < n_single < R and _SPLIT_MIXED:
        order = [i for i in range(R) if lens[i] == 1] + [i for i in range(R) if lens[i] != 1]
        place = [0] * R
        for new_i, old_i in enumerate(order):
            place[old_i] = new_i
        want_order = place                      # the caller's entry i is entry place[i] of the step
        entries = [entries[i] for i in order]
        lens, starts, slots = [lens[i] for i in order], [starts[i] for i in order], [slots[i] for i in order]
    n_want = sum(len(e.want) for e in entries)
    max_blocks = [max(1, max(len(e.cache.tables[g]) for e in entries)) for g in range(len(cache.pools))]
    lay = MetaLayout(T, R, n_want, max_blocks)
    host = torch.empty(lay.total, dtype=torch.int32, pin_memory=torch.device(device).type == "cuda")
    cu, _ = fill(host.numpy(), lay, entries, cache, lens, starts, slots, vocab_size, want_order)
    dev = host.to(device, non_blocking=True)
    ctx = lay.context(dev, cache, device)
    ctx.host_cu_tokens = [int(c) for c in cu]
    ctx.host_start_pos = list(starts)
    ctx.host_state_slots = list(slots)
    ctx.max_portion = max(lens)
    ctx.max_context = max(s + n for s, n in zip(starts, lens))
    ctx.all_decode = T == R
    if want_order is not None:
        ctx.num_decode = n_single
        ctx.decode_max_context = max(starts[i] + 1 for i in range(n_single))
    ctx._host_buffer = host  # keep the pinned buffer alive until the copy has run
    return ctx
