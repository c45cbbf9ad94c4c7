"""Command line in the manner of the reference's gpu_decoder_main (gpu_main.cu:12-71):

    decoder_main <model> [max_batch] [max_prefill_len] [max_prefill_step] [max_total_tokens] [enable_prefix_cache]

with the same positional arguments, defaults (64, 4096, 512, 4096, 1) and meanings.
Prompts are read from standard input, one per line, until an empty line or the end of
input (gpu_main.cu:50-57); a prompt is a list of token ids separated by spaces or
commas, since the tokenizer is outside this engine.  Each request's generated ids are
printed, then the total tokens per second (decoder.cpp:244-251).  What the reference
fixes in its main (temperature 0, top_k 30, 256 new tokens, seed 42; gpu_main.cu:45-48)
are named options here with those defaults.
"""
from __future__ import annotations

import argparse
import re
import sys
import time


def parse_prompt(line: str):
    return [int(t) for t in re.split(r"[,\s]+", line.strip()) if t]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="decoder_main", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model", help="folder with config.json and model.safetensors")
    ap.add_argument("max_batch", nargs="?", type=int, default=64)
    ap.add_argument("max_prefill_len", nargs="?", type=int, default=4096)
    ap.add_argument("max_prefill_step", nargs="?", type=int, default=512)
    ap.add_argument("max_total_tokens", nargs="?", type=int, default=4096)
    ap.add_argument("enable_prefix_cache", nargs="?", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=30)
    ap.add_argument("--max-new-tokens", type=int, default=256)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--no-run-ahead", action="store_true",
                    help="read every step's tokens before the next step is launched")
    args = ap.parse_args(argv)

    print(f"max_batch={args.max_batch} max_total_tokens={args.max_total_tokens} "
          f"max_prefill_len={args.max_prefill_len} max_prefill_step={args.max_prefill_step} "
          f"enable_prefix_cache={args.enable_prefix_cache}", file=sys.stderr)

    prompts = []
    interactive = sys.stdin.isatty()
    while True:
        if interactive:
            print(f"User[{len(prompts)}] token ids (empty to start): ", end="", flush=True)
        line = sys.stdin.readline()
        if not line or not line.strip():
            break
        prompts.append(parse_prompt(line))
    if not prompts:
        print("no input", file=sys.stderr)
        return 1
    print(f"{len(prompts)} requests", file=sys.stderr)

    from .engine import Engine
    from .scheduler import SamplingParams
    engine = Engine(args.model, dtype=args.dtype, device=args.device, max_batch=args.max_batch,
                    max_prefill_len=args.max_prefill_len, max_prefill_tokens_per_step=args.max_prefill_step,
                    max_total_tokens=args.max_total_tokens, page_size=args.page_size, num_pages=args.num_pages,
                    enable_prefix_cache=bool(args.enable_prefix_cache), run_ahead=not args.no_run_ahead)
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k,
                            max_new_tokens=args.max_new_tokens, seed=args.seed, ignore_eos=args.ignore_eos)
    t0 = time.time()
    reqs = [engine.add_request(p, params) for p in prompts]
    while engine.has_work():
        engine.step()
    dt = time.time() - t0
    total = 0
    for i, r in enumerate(reqs):
        print(f"[{i}] ({r.finish_reason}) " + " ".join(map(str, r.output)))
        total += len(r.output)
    print(f"total tokens: {total}, time: {dt:.2f}s, speed: {total / max(dt, 1e-9):.2f} tokens/s", file=sys.stderr)
    return 0
