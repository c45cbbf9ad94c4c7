"""The decode step of a few tokens as ONE kernel launch (``csrc/decode_fused.cu``); opt-in.

The unfused path launches about nine short kernels per layer, each waiting for the one
before.  When every layer of the schedule is the common composition -- pre-norm block,
grouped query attention with one rotary table, SwiGLU, RMSNorm, bfloat16 -- and the step
holds at most 16 single tokens, the model can hand the whole step to one cooperative
kernel.  Measured, that kernel is slower than the unfused path with programmatic
dependent launch (its grid barriers cost what the kernel boundaries cost), so it runs only
with ``QD_FUSED_DECODE=1`` in the environment; it stays as the base for further work and
as a second implementation that the tests compare the first with.

Parts stay ignorant of it: a block that can take part answers ``native_params()``
with its tensors and constants (None otherwise, the default), and this module only
collects the answers.  A model with any other part keeps the unfused path.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from .. import kernels

MAX_TOKENS = 16
_ENABLED = os.environ.get("QD_FUSED_DECODE", "0") == "1"
_TARGET_CTAS = 296


def attention_splits(n_token_heads: int, max_keys: int) -> int:
    """CTAs per (token, kv head): enough items for every resident CTA, but none with fewer than
    eight 16-key chunks (one per warp)."""
    by_fill = max(1, _TARGET_CTAS // max(1, n_token_heads))      # no CTA with two items
    by_work = max(1, (max_keys + 127) // 128)
    return max(1, min(by_fill, by_work, 64))


class FusedDecode:
    """Collected tensors of a model whose decode step the fused kernel can run."""

    def __init__(self, model, entries, common):
        # the model's tensors, not the model: the model refers to this object
        self.embedding = model.embedding
        self.vocab_size = model.vocab_size
        self.lm_head_weight = model.lm_head.weight
        self.entries = entries            # per schedule entry: dict of the block's answer
        self.common = common
        self.device = model.device
        self._cache_id = None
        self.timeline: Optional[torch.Tensor] = None     # int64 [(L + 1) * 16] to have CTA 0 stamp the phases
        self._layers_dev: Optional[torch.Tensor] = None
        dev = self.device
        self.barrier = torch.zeros(2, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.host_status = torch.zeros(1, dtype=torch.int32, pin_memory=True)   # the kernel writes it on failure
        self.attn_tickets = torch.zeros(4096, dtype=torch.int32, device=dev)
        self.n_gemm_tickets = 8192
        self.gemm_tickets = torch.zeros(self.n_gemm_tickets, dtype=torch.int32, device=dev)
        c = common
        n_qkv = (c["H"] + 2 * c["G"]) * c["d"]
        unit = lambda rows, k: -(-rows // 16) * -(-k // 1024)
        most = max(unit(n_qkv, c["D"]), unit(c["D"], c["H"] * c["d"]), unit(c["D"], c["F"]))
        self.scratch_floats = most * 16 * 16
        self.scratch = torch.empty(self.scratch_floats, dtype=torch.float32, device=dev)

    # ---- eligibility ---------------------------------------------------------
    @classmethod
    def try_build(cls, model, force: bool = False) -> Optional["FusedDecode"]:
        """The fused step for ``model`` if its parts allow it and it is switched on (or ``force``)."""
        if not (_ENABLED or force) or model.dtype != torch.bfloat16:
            return None
        entries, common = [], None
        for e in model.schedule:
            if e.cache_of is not None:
                return None
            answer = getattr(model.layers[e.layer], "native_params", lambda: None)()
            if answer is None:
                return None
            key = {k: answer[k] for k in ("D", "H", "G", "d", "F", "window", "scale", "rotary_dim", "pairing")}
            key["position"] = id(answer["position"])
            if common is None:
                common = dict(key, position_obj=answer["position"])
            elif any(common[k] != v for k, v in key.items()):
                return None
            entries.append(answer)
        if common is None or model.hidden_size != common["D"]:
            return None
        final = getattr(model.final_norm, "native_params", lambda: None)()
        if final is None or model.lm_head.bias is not None:
            return None
        c = common
        if c["d"] not in (16, 32, 48, 64, 96, 128) or c["H"] // c["G"] > 16 or c["D"] % 8 or c["F"] % 8 \
                or (c["H"] * c["d"]) % 8:
            return None
        if not kernels.fused_decode_struct_sizes_match():
            raise kernels.KernelError("decode_fused: the argument structures of the library and of the "
                                      "Python side differ in size")
        common["final"] = final
        return cls(model, entries, common)

    def takes(self, ctx) -> bool:
        layout = ctx.cache.layout
        return (ctx.all_decode and ctx.num_tokens <= MAX_TOKENS and ctx.num_wanted == ctx.num_tokens
                and len(layout.groups) == 1 and not layout.fixed and ctx.cache.page_size % 16 == 0
                and ctx.cache.dtype == torch.bfloat16)

    # ---- the step --------------------------------------------------------------
    def _layers(self, cache) -> torch.Tensor:
        if self._cache_id != id(cache):
            arr = (kernels.FusedLayer * len(self.entries))()
            for i, a in enumerate(self.entries):
                arr[i].norm1_w = a["norm1_w"].data_ptr(); arr[i].eps1 = a["eps1"]
                arr[i].wqkv = a["wqkv"].data_ptr()
                arr[i].bqkv = a["bqkv"].data_ptr() if a["bqkv"] is not None else None
                arr[i].wo = a["wo"].data_ptr()
                arr[i].norm2_w = a["norm2_w"].data_ptr(); arr[i].eps2 = a["eps2"]
                arr[i].wgu = a["wgu"].data_ptr()
                arr[i].wd = a["wd"].data_ptr()
                arr[i].kv = cache.layer_kv(i).data_ptr()
            raw = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
            self._layers_dev = raw.to(self.device)
            self._cache_id = id(cache)
        return self._layers_dev

    def forward(self, ctx) -> torch.Tensor:
        c, dev = self.common, self.device
        T, D, H, G, d, F = ctx.num_tokens, c["D"], c["H"], c["G"], c["d"], c["F"]
        V = self.vocab_size
        x = torch.empty((T, D), dtype=torch.float32, device=dev)
        kernels.embedding(x, self.embedding, ctx.tokens)
        window = c["window"] or 0
        splits = attention_splits(T * G, min(ctx.max_context, window or ctx.max_context))
        qkv = torch.empty((T, (H + 2 * G) * d), dtype=torch.float32, device=dev)
        attn_out = torch.empty((T, H * d), dtype=torch.bfloat16, device=dev)
        h = torch.empty((T, F), dtype=torch.bfloat16, device=dev)
        part_o = torch.empty((T * H * splits, d), dtype=torch.float32, device=dev)
        part_ml = torch.empty((T * H * splits, 2), dtype=torch.float32, device=dev)
        logits = torch.empty((T, V), dtype=torch.float32, device=dev)
        grp = ctx.groups[0]
        pos = c["position_obj"]
        p = kernels.FusedParams()
        p.T, p.D, p.H, p.G, p.d, p.F, p.V, p.L = T, D, H, G, d, F, V, len(self.entries)
        p.x, p.qkv, p.attn_out, p.h = x.data_ptr(), qkv.data_ptr(), attn_out.data_ptr(), h.data_ptr()
        p.part_o, p.part_ml, p.tickets = part_o.data_ptr(), part_ml.data_ptr(), self.attn_tickets.data_ptr()
        p.scratch, p.gemm_tickets = self.scratch.data_ptr(), self.gemm_tickets.data_ptr()
        p.scratch_floats, p.n_gemm_tickets = self.scratch_floats, self.n_gemm_tickets
        p.positions, p.token_req = ctx.positions.data_ptr(), ctx.token_request.data_ptr()
        p.block_table, p.slot_map = grp.block_table.data_ptr(), grp.slot_map.data_ptr()
        p.max_blocks, p.page_size, p.splits, p.window = grp.block_table.shape[1], grp.page_size, splits, window
        if pos is not None:
            p.cos_t, p.sin_t = pos.cos.data_ptr(), pos.sin.data_ptr()
        p.rotary_dim, p.pairing = c["rotary_dim"], c["pairing"]
        p.scale_log2e = c["scale"] * math.log2(math.e)
        p.layers = self._layers(ctx.cache).data_ptr()
        fin = c["final"]
        p.final_w, p.final_eps = fin["weight"].data_ptr(), fin["eps"]
        p.lm_head, p.logits = self.lm_head_weight.data_ptr(), logits.data_ptr()
        p.barrier, p.status = self.barrier.data_ptr(), self.status.data_ptr()
        p.host_status = self.host_status.data_ptr()
        if self.timeline is not None:
            p.timeline = self.timeline.data_ptr()
        self.check_status()
        if T * G > self.attn_tickets.numel():
            raise kernels.KernelError("decode_fused: more (token, kv head) pairs than tickets")
        kernels.decode_step_fused(p)
        return logits

    def check_status(self) -> None:
        """Raise if a grid barrier of an earlier launch gave up waiting (results were wrong then)."""
        if int(self.host_status[0]) != 0:
            self.host_status.zero_()
            self.status.zero_()
            self.barrier.zero_()
            raise kernels.KernelError("decode_fused: a grid barrier ran out of time; the step's results are invalid")
