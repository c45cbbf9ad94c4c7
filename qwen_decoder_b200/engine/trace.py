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

PAGE_SIZE = 16
MAX_LIVE = 8


def pool_pages(max_tokens: int, page_size: int = PAGE_SIZE) -> int:
    """Pages for ``max_tokens`` held at once (each request's count a multiple of 64, so of the page)."""
    return max(1, (max_tokens + page_size - 1) // page_size)


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
                with open(os.path.join(out_dir, f"{step['step']}.f32"), "wb") as f:
                    f.write(arr.tobytes())
        for rid in step.get("end", []):
            rc = live.pop(str(rid), None)
            if rc is not None:
                runner.close(rc)
        done.write(f"done {step['step']}\n")
        done.flush()
        n_steps += 1
    return n_steps


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the <step>.f32 files go to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (sizes the cache pool)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    runner = ModelRunner.from_folder(args.model, dtype=args.dtype, device=args.device,
                                     num_pages=pool_pages(args.max_tokens), page_size=PAGE_SIZE,
                                     max_requests=MAX_LIVE)
    replay(runner, sys.stdin, args.out, sys.stdout)
    return 0
