"""Trace replay: feed given token ids through a model step by step and write logits.

Nothing is sampled.  Each input line is one step: for each request its next tokens
and the places whose logits are wanted; requests named in ``end`` give back what they
hold after the step.  It drives the same runner, cache and kernels as generation.
The reference has no such program: its generate_continuous always samples
(decoder.cpp:201-223).
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

import numpy as np
import torch

from ..cache import RequestCache
from .batch import StepEntry
from .runner import ModelRunner

DEFAULT_PAGE_SIZE = 16
DEFAULT_MAX_LIVE = 8


def pool_pages(max_tokens: int, page_size: int = DEFAULT_PAGE_SIZE, max_live: int = DEFAULT_MAX_LIVE) -> int:
    """Pages for ``max_tokens`` held at once.  The caller counts each request's tokens rounded up to a
    multiple of 64; a page that is no divisor of 64 rounds each request up to its own size instead, which
    may take up to one page more per live request."""
    pages = (max_tokens + page_size - 1) // page_size
    if 64 % page_size:
        pages += max_live
    return max(1, pages)


def replay(runner: ModelRunner, lines: IO[str], out_dir: str, done: IO[str]) -> int:
    os.makedirs(out_dir, exist_ok=True)
    live: Dict[str, RequestCache] = {}
    n_steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = []
        for e in step.get("entries", []):
            rid = str(e["id"])
            rc = live.get(rid)
            if rc is None:
                rc = live[rid] = runner.open(rid)
            entries.append(StepEntry(rc, [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                arr = logits.to("cpu").numpy().astype("<f4", copy=False)
                runner.check_status()        # logits of a step in which a kernel's wait ran out are not written
                with open(os.path.join(out_dir, f"{step['step']}.f32"), "wb") as f:
                    f.write(arr.tobytes())
        for rid in step.get("end", []):
            rc = live.pop(str(rid), None)
            if rc is not None:
                runner.close(rc)
        done.write(f"done {step['step']}\n")
        done.flush()
        n_steps += 1
    runner.check_status()
    return n_steps


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the <step>.f32 files go to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (sizes the cache pool)")
    ap.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE,
                    help="tokens in a page of the cache (a multiple of 16 for the bfloat16 kernels)")
    ap.add_argument("--max-live", type=int, default=DEFAULT_MAX_LIVE, help="most requests live at a time")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.page_size < 1 or args.max_live < 1:
        ap.error("--page-size and --max-live must be at least 1")
    runner = ModelRunner.from_folder(args.model, dtype=args.dtype, device=args.device,
                                     num_pages=pool_pages(args.max_tokens, args.page_size, args.max_live),
                                     page_size=args.page_size, max_requests=args.max_live)
    replay(runner, sys.stdin, args.out, sys.stdout)
    return 0
