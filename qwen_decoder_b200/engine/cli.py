"""Command line in the manner of the reference's gpu_decoder_main (gpu_main.cu:12-71):

    decoder_main <model> [max_batch] [max_prefill_len] [max_prefill_step] [max_total_tokens] [enable_prefix_cache]

with the same positional arguments, defaults (64, 4096, 512, 4096, 1) and meanings.
Prompts are read from standard input, one per line, until an empty line or the end of
input (gpu_main.cu:50-57); a prompt is a list of token ids separated by spaces or
commas, since the tokenizer is outside this engine.  Each request's generated ids are
printed, then the total tokens per second (decoder.cpp:244-251).  What the reference
fixes in its main (temperature 0, top_k 30, 256 new tokens, seed 42; gpu_main.cu:45-48)
are named options here with those defaults.  Beyond the reference's: ``--random-weights`` (the model
folder needs config.json only; weights N(0, 0.02) from ``--weights-seed`` are made on the device),
``--prompt-ids`` / ``--prompt-file`` / ``--random-prompts`` instead of standard input, and ``--stats``:
one line per step as the reference prints it (decoder.cpp:178-185: tokens, decoding and prefilling
requests, prompt tokens) with the step's device time and the free pages, and prompt and decode
tokens per second apart at the end.
"""
from __future__ import annotations

import argparse
import re
import sys
import time


def parse_prompt(line: str):
    return [int(t) for t in re.split(r"[,\s]+", line.strip()) if t]


def random_prompts(spec: str, length: str, vocab_size: int, seed: int):
    """``spec`` prompts of uniform random ids; ``length`` = "A" or "A:B" (uniform in [A, B])."""
    import random
    rng = random.Random(seed)
    lo, _, hi = length.partition(":")
    lo, hi = int(lo), int(hi or lo)
    return [[rng.randrange(vocab_size) for _ in range(rng.randint(lo, hi))] for _ in range(int(spec))]


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
    ap.add_argument("--random-weights", action="store_true",
                    help="the folder holds config.json only; random weights are made on the device")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of --random-weights")
    ap.add_argument("--prompt-ids", action="append", default=[], metavar="IDS",
                    help='a prompt as token ids, "1,2,3" (repeatable); no prompts are read from standard input then')
    ap.add_argument("--prompt-file", default=None, help="a file with one prompt (token ids) per line")
    ap.add_argument("--random-prompts", default=None, metavar="N", help="N prompts of uniform random token ids")
    ap.add_argument("--len", dest="length", default="128", metavar="A[:B]",
                    help="length of the random prompts, or a range to draw each from")
    ap.add_argument("--stats", action="store_true", help="a line per step, and prompt / decode tokens per second")
    args = ap.parse_args(argv)

    print(f"max_batch={args.max_batch} max_total_tokens={args.max_total_tokens} "
          f"max_prefill_len={args.max_prefill_len} max_prefill_step={args.max_prefill_step} "
          f"enable_prefix_cache={args.enable_prefix_cache}", file=sys.stderr)

    from ..config import load_config
    from .engine import Engine
    from .scheduler import SamplingParams
    prompts = [parse_prompt(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [parse_prompt(line) for line in f if line.strip()]
    if args.random_prompts:
        prompts += random_prompts(args.random_prompts, args.length, load_config(args.model).vocab_size, args.seed)
    if not (args.prompt_ids or args.prompt_file or args.random_prompts):
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

    options = dict(dtype=args.dtype, device=args.device, max_batch=args.max_batch,
                   max_prefill_len=args.max_prefill_len, max_prefill_tokens_per_step=args.max_prefill_step,
                   max_total_tokens=args.max_total_tokens, page_size=args.page_size, num_pages=args.num_pages,
                   enable_prefix_cache=bool(args.enable_prefix_cache), run_ahead=not args.no_run_ahead,
                   record_steps=args.stats)
    if args.random_weights:
        engine = Engine(config=load_config(args.model), random_seed=args.weights_seed, **options)
    else:
        engine = Engine(args.model, **options)
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
    if args.stats:
        recs = engine.step_records()
        for r in recs:
            print(f"step {r['step']}: total_tokens={r['tokens']} n_decode={r['decode_tokens']} "
                  f"n_prefill={r['prompt_requests']} prefill_tokens={r['prompt_tokens']} ms={r['ms']:.3f} "
                  f"pages_free={min(r['pages_free']) if r['pages_free'] else 0} running={r['running']} "
                  f"waiting={r['waiting']}{' ahead' if r['planned_ahead'] else ''}", file=sys.stderr)
        # a step's time goes to prompt and decode tokens in proportion to their numbers
        p_tok = sum(r["prompt_tokens"] for r in recs)
        d_tok = sum(r["decode_tokens"] for r in recs)
        p_ms = sum(r["ms"] * r["prompt_tokens"] / r["tokens"] for r in recs if r["tokens"])
        d_ms = sum(r["ms"] * r["decode_tokens"] / r["tokens"] for r in recs if r["tokens"])
        st = engine.stats
        print(f"prompt: {p_tok} tokens, {p_tok / max(p_ms, 1e-9) * 1e3:.1f} tokens/s; decode: {d_tok} tokens, "
              f"{d_tok / max(d_ms, 1e-9) * 1e3:.1f} tokens/s (device time of the steps); steps {len(recs)}, "
              f"preemptions {st.get('preemptions', 0)}, prefix-cache hit tokens {st.get('prefix_hit_tokens', 0)}",
              file=sys.stderr)
    return 0
