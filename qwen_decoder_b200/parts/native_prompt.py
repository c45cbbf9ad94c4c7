"""The layers of a prompt step launched from native code (``csrc/prompt_exec.cu``).

A step with a prompt portion is launched kernel by kernel.  From Python that is about
15 us of host time per launch, 5 ms for 36 layers, while the device needs 3 ms for a
portion of 512 tokens: the device waits for the interpreter.  When every layer of the
schedule is the common composition -- pre-norm block, grouped-query attention with one
rotary table, SwiGLU, RMSNorm, bfloat16 -- the same launchers are called,
in the same order and with the same arguments, from one C++ loop instead.  The embedding
before it and the output projection after it stay with the model.

Parts stay ignorant of it: a block that can take part answers ``native_params()``
with its tensors and constants (None otherwise, the default), and this module only
collects the answers.  A model with any other part or another dtype keeps the parts' own
path, and so does a step of single tokens (it replays as a CUDA graph); so does everything
when ``QD_NATIVE_PROMPT=0`` is set.

One difference in arithmetic: the parts' q/k/v product adds its bias in the product's
epilogue, here the rotation kernel adds it to the product's bfloat16 output (one more
rounding to bfloat16 of q, k and v).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import kernels
from . import matmul_backend

_ENABLED = os.environ.get("QD_NATIVE_PROMPT", "1") != "0"
_MIN_TOKENS = 1       # measured faster at every length: 4 tokens 3.2 against 4.4 ms
# the one arrangement of parts whose order of kernels csrc/prompt_exec.cu restates: a block that answers
# ``native_params()`` with any other ``composition`` (another order, another part) keeps the parts' own path
COMPOSITION = "pre_norm/gq_attention/swiglu/rmsnorm/rmsnorm"
OWN_LAUNCHES_PER_LAYER = 5    # norm, rotation, attention, norm, SwiGLU; the four products are the library's


class NativePrompt:
    """Collected tensors of a model whose prompt steps the native loop can run."""

    def __init__(self, model, entries, common):
        # the model's tensors, not the model: the model refers to this object
        self.entries = entries            # per schedule entry: dict of the block's answer
        self.common = common
        self.device = model.device
        self.schedule = [e.cache_of is None for e in model.schedule]
        self._cache_id = None
        self._layers = None               # host array of PromptLayer, kept alive here
        self.steps = 0                    # steps run here (tests look at it)

    # ---- eligibility ---------------------------------------------------------
    @classmethod
    def try_build(cls, model) -> Optional["NativePrompt"]:
        if not _ENABLED or model.dtype != torch.bfloat16 or matmul_backend.mode not in ("auto", "cublas") \
                or model.device.type != "cuda":
            return None
        entries, common = [], None
        for e in model.schedule:
            answer = getattr(model.layers[e.layer], "native_params", lambda: None)()
            if answer is None or answer.get("composition") != COMPOSITION:
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
        if final is None or final.get("kind") != "rmsnorm" or "weight" not in final:
            return None
        c = common
        n_qkv = (c["H"] + 2 * c["G"]) * c["d"]
        # what the vectorized rotation kernel and the library product take
        if c["pairing"] not in (0, 1) or c["rotary_dim"] % (8 if c["pairing"] == 0 else 16):
            return None
        if c["d"] % 8 or c["D"] % 8 or c["F"] % 8 or n_qkv % 8:
            return None
        if not kernels.prompt_exec_struct_sizes_match():
            raise kernels.KernelError("prompt_exec: the argument structures of the library and of the "
                                      "Python side differ in size")
        common["final"] = final
        return cls(model, entries, common)

    def attention_impl(self, page_size: int) -> Optional[int]:
        """1: tcgen05 kernel, 0: mma.sync kernel, None: neither takes these sizes."""
        c = self.common
        if kernels.prefill_tc5_supported(torch.bfloat16, c["H"], c["G"], c["d"], page_size) \
                and os.environ.get("QD_PREFILL_TC5", "1") != "0":
            return 1
        if kernels.flash_prefill_supported(torch.bfloat16, c["H"], c["G"], c["d"], page_size):
            return 0
        return None

    def takes(self, ctx) -> bool:
        layout = ctx.cache.layout
        return (not ctx.all_decode and ctx.num_tokens >= _MIN_TOKENS
                and len(layout.groups) == 1 and not layout.fixed and ctx.cache.dtype == torch.bfloat16
                and self.attention_impl(ctx.cache.page_size) is not None)

    # ---- the step --------------------------------------------------------------
    def _layer_array(self, cache):
        if self._cache_id != id(cache):
            arr = (kernels.PromptLayer * len(self.entries))()
            for i, a in enumerate(self.entries):
                arr[i].norm1_w = a["norm1_w"].data_ptr(); arr[i].eps1 = a["eps1"]
                arr[i].norm2_w = a["norm2_w"].data_ptr(); arr[i].eps2 = a["eps2"]
                arr[i].wqkv = a["wqkv"].data_ptr()
                arr[i].bqkv = a["bqkv"].data_ptr() if a["bqkv"] is not None else None
                arr[i].wo = a["wo"].data_ptr()
                arr[i].wgu = a["wgu"].data_ptr()
                arr[i].wd = a["wd"].data_ptr()
                arr[i].kv = cache.layer_kv(i).data_ptr()
                arr[i].write_kv = 1 if self.schedule[i] else 0
            self._layers, self._cache_id = arr, id(cache)
        return self._layers

    def forward(self, ctx, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Runs every layer on the residual sum ``x`` (float32 [T, D], the embeddings on entry) and returns
        the normalised rows at the wanted places (bfloat16 [n_wanted, D]; None if nothing is wanted)."""
        c, dev = self.common, self.device
        T, D, H, G, d, F = ctx.num_tokens, c["D"], c["H"], c["G"], c["d"], c["F"]
        bf = torch.bfloat16
        n_qkv = (H + 2 * G) * d
        # one scratch buffer for the step, carved into the six activations (all offsets 16-byte aligned)
        sizes = [T * D, T * n_qkv, T * H * d, T * D, T * 2 * F, T * F]
        offs, total = [], 0
        for n in sizes:
            offs.append(total)
            total += (n + 7) // 8 * 8
        scratch = torch.empty(total, dtype=bf, device=dev)
        base = scratch.data_ptr()
        hrows = torch.empty((ctx.num_wanted, D), dtype=bf, device=dev) if ctx.num_wanted else None
        group = ctx.groups[0]
        pos = c["position_obj"]
        p = kernels.PromptParams()
        use_tc5 = self.attention_impl(group.page_size)
        # a mixed step: its single tokens (first in the batch) go to the split-KV decode kernel
        nd = ctx.num_decode if kernels.flash_decode_supported(bf, H, G, d, group.page_size) else 0
        p.fn = kernels.prompt_fns(bool(use_tc5), nd > 0)
        keep = None
        if nd:
            from .attention import decode_splits
            window = c["window"] or 0
            p.n_decode = nd
            p.decode_splits = decode_splits(nd * G, min(ctx.decode_max_context, window or ctx.decode_max_context))
            keep = kernels.decode_scratch(nd, H, d, G, p.decode_splits, dev)
            p.token_req = ctx.token_request.data_ptr()
            p.part_o, p.part_ml, p.tickets = (t.data_ptr() if t is not None else None for t in keep)
        p.fn.blas = torch.cuda.current_blas_handle()
        p.layers = ctypes.cast(self._layer_array(ctx.cache), ctypes.c_void_p)
        p.n_layers = len(self.entries)
        p.T, p.R, p.D, p.H, p.G, p.d, p.F = T, ctx.num_requests, D, H, G, d, F
        p.page_size, p.window = group.page_size, c["window"] or 0
        p.rotary_dim, p.pairing = c["rotary_dim"], c["pairing"]
        p.max_blocks = group.block_table.shape[1]
        p.use_tc5 = use_tc5
        p.n_wanted = ctx.num_wanted
        p.scale, p.final_eps = c["scale"], c["final"]["eps"]
        p.n_pages = ctx.cache.layer_kv(0).shape[0]
        p.positions, p.slot_map = ctx.positions.data_ptr(), group.slot_map.data_ptr()
        p.block_table = group.block_table.data_ptr()
        p.cu_tokens, p.start_pos = ctx.cu_tokens.data_ptr(), ctx.start_pos.data_ptr()
        p.logit_rows = ctx.logit_rows.data_ptr() if ctx.num_wanted else None
        p.cos_t = pos.cos.data_ptr() if pos is not None and c["rotary_dim"] else None
        p.sin_t = pos.sin.data_ptr() if pos is not None and c["rotary_dim"] else None
        p.final_w = c["final"]["weight"].data_ptr()
        p.x, p.delta0 = x.data_ptr(), None
        p.h, p.qkv, p.attn, p.delta, p.gu, p.act = (base + 2 * o for o in offs)
        p.hrows = hrows.data_ptr() if hrows is not None else None
        shares = matmul_backend.library_shares(T, D, F)
        down_part = torch.empty((shares, T, D), dtype=torch.float32, device=dev) if shares else None
        p.down_shares = shares
        p.down_part = down_part.data_ptr() if shares else None
        n_launches = len(self.entries) * (OWN_LAUNCHES_PER_LAYER + (1 if nd else 0)) + (1 if ctx.num_wanted else 0)
        kernels.prompt_exec(p, n_launches)
        self.steps += 1
        matmul_backend.counters["library"] += 4 * len(self.entries)
        return hrows
