#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, at the Qwen2.5-3B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A step is one decode step of a batch of requests that each hold ``--context`` cached
tokens.  Prints ONE JSON line: ``value`` = decoded tokens per second (device-timed
with CUDA events over exactly K steps after W warm-up steps), ``e2e`` = the same
through the Python entry point (``Engine.step``: host token ids in through pinned
memory, sampled ids back to the host, every step), ``prefill`` = a 2,048-token
prompt in one step, ``roofline`` = bytes a decode step must read / its time against
the measured copy bandwidth, ``points`` = decode at batch 1 and 64 and prompts of 128
and 512 tokens in one step (tokens per second, host launching included).

Weights are random (N(0, 0.02), seeded); the caches of the decode requests are filled
with random values instead of running 2,048-token prompts first (decode time does not
depend on the values).  Nothing needs flushing between steps: a step streams all
weights (6.2 GB), far more than the 126 MB L2.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE_3B = dict(
    architectures=["Qwen2ForCausalLM"], hidden_size=2048, intermediate_size=11008, num_hidden_layers=36,
    num_attention_heads=16, num_key_value_heads=2, vocab_size=151936, max_position_embeddings=32768,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
# the two other GPU-sized shapes (their own workloads: --micro serve, and --batch/--context for long contexts)
SHAPE_7B = dict(
    architectures=["Qwen2ForCausalLM"], hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
    num_attention_heads=28, num_key_value_heads=4, vocab_size=152064, max_position_embeddings=32768,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
SHAPE_32B = dict(
    architectures=["Qwen2ForCausalLM"], hidden_size=5120, intermediate_size=27648, num_hidden_layers=64,
    num_attention_heads=40, num_key_value_heads=8, vocab_size=152064, max_position_embeddings=32768,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
SHAPES = {"3B": SHAPE_3B, "7B": SHAPE_7B, "32B": SHAPE_32B}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            return out, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def decode_bytes(cfg, layers, batch, ctx_mean):
    D, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, G = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = D // H
    per_layer = (H * d + 2 * G * d) * D + D * H * d + 3 * F * D
    weights = (layers * per_layer + V * D) * 2          # every matrix once; the output matrix (tied or not) once
    kv = batch * ctx_mean * layers * 2 * G * d * 2
    return weights + kv


def prefill_flops(cfg, layers, T):
    D, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, G = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = D // H
    per_layer = (H * d + 2 * G * d) * D + D * H * d + 3 * F * D
    attn = 4 * d * H * (T * (T + 1) // 2)               # QK^T and PV over the causal triangle
    return layers * (2 * T * per_layer + attn) + 2 * V * D


def serve(args):
    """A whole serving run through the entry point: ``--batch`` requests arrive at once, each with a random
    prompt of ``--context`` tokens (or, with ``--context-range A:B``, of a length drawn uniformly from [A, B])
    and generate ``--steps`` tokens each (greedy, no stop token); continuous batching, prompt portions of at
    most ``--prefill-budget`` tokens a step mixed with decode tokens (the reference's loop: decoder.cpp:35-239,
    its budget decoder.cpp:90-96).  Wall clock of the second round, and from the engine's step records the
    device time of its steps: prompt and output tokens per second and the spread of the step times."""
    import random
    import torch
    from qwen_decoder_b200 import kernels
    from qwen_decoder_b200.config import Qwen2Config
    from qwen_decoder_b200.engine import Engine, SamplingParams
    shape = SHAPES[args.shape]
    cfg = Qwen2Config.from_dict(dict(shape, num_hidden_layers=args.layers))
    n, new = args.batch, args.steps
    lo, hi = args.context, args.context
    if args.context_range:
        a, _, b = args.context_range.partition(":")
        lo, hi = int(a), int(b or a)
    page = args.page_size
    rng = random.Random(3)
    lengths = [[rng.randint(lo, hi) for _ in range(n)] for _ in range(2)]
    most = max(sum((p + new + page) // page + 1 for p in ls) for ls in lengths)
    engine = Engine(config=cfg, random_seed=0, dtype="bfloat16", device="cuda:0", max_batch=max(64, n),
                    max_prefill_len=1 << 20, page_size=page, num_pages=most + 64,
                    max_positions=hi + new + 64, max_prefill_tokens_per_step=args.prefill_budget,
                    max_total_tokens=max(4096, args.prefill_budget + n), record_steps=True)
    gen = torch.Generator().manual_seed(3)
    sp = SamplingParams(max_new_tokens=new, ignore_eos=True)
    rounds = []
    for rnd in range(2):                 # the first round builds libraries and captures graphs
        prompts = [torch.randint(0, cfg.vocab_size, (p,), generator=gen).tolist() for p in lengths[rnd]]
        torch.cuda.synchronize()
        r0 = len(engine.step_records())
        s0, l0, t0 = engine.runner.steps, kernels.launches(), time.perf_counter()
        g0 = len(engine.runner._graphs)
        outs = engine.generate(prompts, sp)
        torch.cuda.synchronize()
        rounds.append((time.perf_counter() - t0, engine.runner.steps - s0, kernels.launches() - l0,
                       sum(len(o) for o in outs), engine.step_records()[r0:], len(engine.runner._graphs) - g0))
    sec, steps, launches, made, recs, new_graphs = rounds[-1]
    n_prompt = sum(lengths[1])
    pct = lambda xs, q: round(sorted(xs)[min(len(xs) - 1, int(q * len(xs)))], 3) if xs else None
    mixed = [r["ms"] for r in recs if r["prompt_tokens"] and r["decode_tokens"]]
    prompt_only = [r["ms"] for r in recs if r["prompt_tokens"] and not r["decode_tokens"]]
    decode_only = [r["ms"] for r in recs if not r["prompt_tokens"]]
    print(json.dumps({"micro": "serve", "shape": args.shape, "requests": n,
                      "prompt_tokens": n_prompt, "prompt_lengths": [lo, hi], "new_tokens": new,
                      "prefill_budget": args.prefill_budget, "layers": args.layers, "layers_full": shape["num_hidden_layers"],
                      "seconds": round(sec, 4), "engine_steps": steps, "generated": made,
                      "prompt_tok_s": round(n_prompt / sec, 1), "generated_tok_s": round(made / sec, 1),
                      "total_tok_s": round((made + n_prompt) / sec, 1), "gpu_launches": launches,
                      "step_ms": {"all": {"n": len(recs), "p50": pct([r["ms"] for r in recs], 0.5),
                                          "p90": pct([r["ms"] for r in recs], 0.9), "max": pct([r["ms"] for r in recs], 1.0)},
                                  "prompt_and_decode": {"n": len(mixed), "p50": pct(mixed, 0.5), "p90": pct(mixed, 0.9)},
                                  "prompt_only": {"n": len(prompt_only), "p50": pct(prompt_only, 0.5)},
                                  "decode_only": {"n": len(decode_only), "p50": pct(decode_only, 0.5), "p90": pct(decode_only, 0.9)}},
                      "device_seconds_of_steps": round(sum(r["ms"] for r in recs) / 1e3, 4),
                      "first_round_seconds": round(rounds[0][0], 3),
                      # decode-step shapes (padded batch, block-table width) met for the first time in the timed
                      # round: each is run once eagerly and captured, which is what the slowest steps are
                      "graphs_captured_in_the_timed_round": new_graphs}))
    return 0


def mixed_step(args):
    """One step of a busy server: ``--batch`` decoding requests at ``--context`` cached tokens each beside one
    prompt portion of ``--prefill-tokens`` tokens that follows ``--history`` cached tokens, at ``--shape`` with
    ``--layers`` layers; device time by CUDA events (for launch lists: a few layers are enough)."""
    import torch
    from qwen_decoder_b200.config import Qwen2Config
    from qwen_decoder_b200.engine import ModelRunner, StepEntry
    cfg = Qwen2Config.from_dict(dict(SHAPES[args.shape], num_hidden_layers=args.layers))
    B, C, P, hist, page = args.batch, args.context, args.prefill_tokens, args.history, args.page_size
    pages = (B * (C + 64) + 16 * (P + hist + 64)) // page + 64
    runner = ModelRunner.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", num_pages=pages, page_size=page,
                                     max_requests=B + 4, max_positions=max(C, P + hist) + 128)
    for kv in runner.cache.kv:
        kv.normal_(0.0, 1.0)
    dec = []
    for i in range(B):
        rc = runner.open(f"d{i}")
        runner.cache.ensure(rc, C)
        runner.cache.commit(rc, C)
        dec.append(rc)
    times = []
    for i in range(max(3, args.warmup) + args.steps):
        rc = runner.open(f"p{i}")
        runner.cache.ensure(rc, hist)
        runner.cache.commit(rc, hist)
        entries = [StepEntry(rc, list(range(P)), [P - 1])] + [StepEntry(d, [7], [0]) for d in dec]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step(entries)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        runner.close(rc)
        for d in dec:                     # the decoding requests stay where they were
            d.num_tokens -= 1
    ts = sorted(times[max(3, args.warmup):])
    print(json.dumps({"micro": "mixed_step", "shape": args.shape, "layers": args.layers, "decoding_requests": B,
                      "context": C, "prompt_tokens": P, "history": hist, "ms": round(ts[len(ts) // 2], 3)}))
    return 0


def micro(args):
    """One kernel alone: W-streaming contraction, decode attention or prefill attention at the 3B sizes."""
    if args.micro == "serve":
        return serve(args)
    if args.micro == "mixed_step":
        return mixed_step(args)
    import math
    import torch
    from qwen_decoder_b200 import kernels
    dev = "cuda:0"
    H, G, d, ps = 16, 2, 128, args.page_size
    T = args.tokens
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if args.micro == "gemm":
        N, K = {"qkv": (2560, 2048), "o": (2048, 2048), "gate_up": (22016, 2048), "down": (2048, 11008),
                "lm_head": (151936, 2048)}[args.micro_shape]
        x = torch.randn(T, K, device=dev).bfloat16()
        if args.micro_graph:
            # launch latency left out: a graph of launches on so many copies of the weights that L2 cannot hold
            # them, replayed; with --micro-splits the product leaves float32 partial sums of that many shares of K
            copies = max(4, int(400e6 // (N * K * 2)) + 1)
            ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(copies)]
            out = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
            sp = args.micro_splits
            part = torch.empty(sp, T, N, device=dev, dtype=torch.float32) if sp > 1 else None
            if args.micro_impl == "cublas":
                one = lambda w: torch.mm(x, w.t(), out=out)
            else:
                kernels.skinny_impl = args.micro_impl
                kernels.TC5_POLICY_TOKENS = kernels.SKINNY_POLICY_TOKENS = 64
                one = (lambda w: kernels._skinny_call(x, w, None, out, None, T, N, K, 1, kernels.EPI_STORE, "micro")) \
                    if sp <= 1 else (lambda w: kernels._skinny_call(x, w, None, None, part, T, N, K, sp, kernels.EPI_PARTIAL, "micro"))
            for w in ws:
                one(w)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for w in ws:
                    one(w)
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(4):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (4 * copies)
            print(json.dumps({"micro": "gemm", "impl": args.micro_impl, "shape": args.micro_shape, "tokens": T,
                              "splits": sp, "us": round(us, 2), "GB/s": round(N * K * 2 / us / 1e3, 1),
                              "note": f"mean of {copies} launches on different weights inside a replayed graph"}))
            return 0
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        out = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
        if args.micro_impl == "cublas":
            run = lambda: torch.mm(x, w.t(), out=out)
        else:
            kernels.skinny_impl = args.micro_impl
            run = lambda: kernels._skinny_call(x, w, None, out, None, T, N, K, 1, kernels.EPI_STORE, "micro")
        work = {"bytes": N * K * 2, "flops": 2 * T * N * K}
    elif args.micro == "decode_attention":
        ctx = args.context + 128
        npg = (ctx + ps - 1) // ps
        kv = torch.randn(T * npg + 4, 2, G, ps, d, device=dev).bfloat16()
        bt = torch.arange(T * npg, dtype=torch.int32, device=dev).view(T, npg).contiguous()
        q = torch.randn(T, H * d, device=dev).bfloat16()
        out = torch.empty(T, H * d, device=dev, dtype=torch.bfloat16)
        tr = torch.arange(T, dtype=torch.int32, device=dev)
        pos = torch.full((T,), ctx - 1, dtype=torch.int32, device=dev)
        from qwen_decoder_b200.parts.attention import decode_splits
        splits = decode_splits(T * G, ctx)
        run = lambda: kernels.decode_attention(q, H * d, out, kv, bt, tr, pos, T, H, G, d, ps, 1 / math.sqrt(d), 0, splits)
        work = {"bytes": T * ctx * 2 * G * d * 2, "flops": 4 * T * ctx * H * d, "splits": splits}
    elif args.micro == "decode_attention_rope":
        # from the float32 partial sums of q, k, v: bias, rotation, cache write and attention in one kernel
        ctx = args.context + 128
        npg = (ctx + ps) // ps
        kv = torch.randn(T * npg + 4, 2, G, ps, d, device=dev).bfloat16()
        bt = torch.arange(T * npg, dtype=torch.int32, device=dev).view(T, npg).contiguous()
        part = torch.randn(2, T, (H + 2 * G) * d, device=dev) * 0.5
        bias = torch.randn((H + 2 * G) * d, device=dev)
        out = torch.empty(T, H * d, device=dev, dtype=torch.bfloat16)
        tr = torch.arange(T, dtype=torch.int32, device=dev)
        pos = torch.full((T,), ctx - 1, dtype=torch.int32, device=dev)
        slots = (bt[:, (ctx - 1) // ps] * ps + (ctx - 1) % ps).to(torch.int32)
        ang = torch.arange(ctx, device=dev, dtype=torch.float32)[:, None] * torch.rand(d // 2, device=dev)[None, :]
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        from qwen_decoder_b200.parts.attention import decode_rope_splits
        splits = decode_rope_splits(T * G, ctx)
        run = lambda: kernels.decode_attention_rope(part, bias, out, kv, bt, tr, pos, slots, H, G, d, ps,
                                                    1 / math.sqrt(d), 0, splits, True, d, 0, cos, sin)
        work = {"bytes": T * ctx * 2 * G * d * 2, "flops": 4 * T * ctx * H * d, "splits": splits}
    else:
        T = args.prefill_tokens
        kv = torch.randn(T // ps + 4, 2, G, ps, d, device=dev).bfloat16()
        bt = torch.arange(T // ps, dtype=torch.int32, device=dev).view(1, -1).contiguous()
        q = torch.randn(T, (H + 2 * G) * d, device=dev).bfloat16()
        out = torch.empty(T, H * d, device=dev, dtype=torch.bfloat16)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        st = torch.tensor([0], dtype=torch.int32, device=dev)
        fn = kernels.prefill_attention if args.micro_impl == "regs" else kernels.prefill_attention_tc5
        run = lambda: fn(q, q.stride(0), out, kv, bt, cu, st, 1, T, H, G, d, ps, 1 / math.sqrt(d), 0)
        work = {"bytes": T * (H + 2 * G) * d * 2 * 2, "flops": 4 * d * H * (T * (T + 1) // 2)}
        if args.timeline and args.micro_impl != "regs" and T >= 2048:
            # nanosecond stamps written by the kernel itself (layout: AtParams::timeline in csrc/attention_tc5.cu): of
            # the CTA whose rows end at key 2047 (16 key tiles) the softmax thread of row 0 and the MMA thread, tile
            # by tile, and that CTA's phases; of every CTA its start, end, SM and number of key tiles.  Each launch is
            # synchronised, so that no CTA starts under the launch before it.
            n_cta = (T // (128 // (H // G)) + 2) * G
            tl = torch.zeros(192 + 4 * n_cta, dtype=torch.int64, device=dev)
            for _ in range(3):
                fn(q, q.stride(0), out, kv, bt, cu, st, 1, T, H, G, d, ps, 1 / math.sqrt(d), 0, tl)
                torch.cuda.synchronize()
            sm, mm = tl[:128].view(16, 8).cpu(), tl[128:192].view(16, 4).cpu()
            t0 = int(sm[0][7])
            us = lambda x: (int(x) - t0) / 1e3
            names_s = ["top", "S ready", "S loaded", "maximum shared", "exponentials", "P stored"]
            names_m = ["top", "P ready", "K, V ready and product issued", "scores of tile + 2 issued"]
            for j in range(16):
                print(f"tile {j:2d}  softmax: " + "  ".join(f"{n} {us(sm[j][i]):.2f}" for i, n in enumerate(names_s)) +
                      "  ||  mma: " + "  ".join(f"{n} {us(mm[j][i]):.2f}" for i, n in enumerate(names_m)), file=sys.stderr)
            phases = ["start", "tensor memory allocated", "request found", "Q stored", "last P stored",
                      "last product complete", "end"]
            print("that CTA: " + "  ".join(f"{n} {us(sm[i][7]):.2f}" for i, n in enumerate(phases)) +
                  f"  output written {us(sm[15][6]):.2f}", file=sys.stderr)
            rec = tl[192:].view(n_cta, 4).cpu()
            rec = rec[rec[:, 0] > 0]
            first = int(rec[:, 0].min())
            fixed = sorted((int(e) - int(s0)) / 1e3 - 1.2 * int(n) for s0, e, _, n in rec.tolist())
            per_sm = {}
            for s0, e, smid, n in rec.tolist():
                per_sm.setdefault(smid, []).append(((s0 - first) / 1e3, (e - first) / 1e3, n))
            last = max(per_sm.values(), key=lambda v: max(x[1] for x in v))
            print(f"{len(rec)} CTAs on {len(per_sm)} SMs; last end {(int(rec[:, 1].max()) - first) / 1e3:.1f} us; "
                  f"a CTA's time minus 1.2 us per key tile: median {fixed[len(fixed) // 2]:.1f} us; "
                  f"the SM that ends last ran (start, end, key tiles): {sorted(last)}", file=sys.stderr)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    ts = []
    for _ in range(20):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); run(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    us = ts[len(ts) // 2]
    print(json.dumps({"micro": args.micro, "impl": args.micro_impl if args.micro == "gemm" else ("mma.sync" if args.micro == "prefill_attention" and args.micro_impl == "regs" else "ours"),
                      "shape": args.micro_shape if args.micro == "gemm" else None, "tokens": T, "us": round(us, 2),
                      "GB/s": round(work["bytes"] / us / 1e3, 1), "TFLOP/s": round(work["flops"] / us / 1e6, 2),
                      "note": "eager launch between CUDA events after an L2 flush; includes ~8 us of launch latency",
                      **{k: v for k, v in work.items() if k == "splits"}}))
    return 0


def reference_arm(args):
    """The same metric from the reference's own program (baseline/reference_arm.py says how it is built and
    fed): decode tokens per second at ``--batch`` with ``--context``-token prompts from its per-step lines,
    batch 1 and 64 and the 2,048-token prompt step beside it.  Its weights are float16 where ours are
    bfloat16: the same bytes per step."""
    import tempfile
    from baseline import reference_arm as ra
    if args.gpus != 1:
        print(f"bench.py: the reference's gpu_decoder_main runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    cfgd = dict(SHAPE_3B, num_hidden_layers=args.layers)
    W = max(3, args.warmup)
    out_dir = os.path.join(ROOT, "gpurun_out")
    try:
        os.makedirs(out_dir, exist_ok=True)
    except OSError:
        out_dir = tempfile.gettempdir()
    clocks = ClockSampler()
    try:
        ra.ensure_binary()
        with tempfile.TemporaryDirectory(prefix="qd_ref_") as tmp:
            model = os.path.join(tmp, "model.gguf")
            ra.write_gguf(model, cfgd, seed=0, context_length=4096)
            clocks.start()
            main_rec = ra.run(model, args.batch, args.context, log_path=os.path.join(out_dir, f"reference_b{args.batch}.log"))
            ck = clocks.stop()
            recs = {args.batch: main_rec}
            if not args.no_points:
                for b in (1, 64):
                    if b not in recs:
                        recs[b] = ra.run(model, b, args.context, log_path=os.path.join(out_dir, f"reference_b{b}.log"))
    except ra.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    ms = main_rec["decode_ms"][W:]
    if not ms:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's run printed no decode steps of the full batch"}))
        return 0
    K = len(ms)
    ms_per_step = sum(ms) / K
    value = args.batch / (ms_per_step / 1e3)
    pk, pk_src = peaks()
    ctx_mean = args.context + W + K / 2.0
    achieved = decode_bytes(cfgd, args.layers, args.batch, ctx_mean) / (ms_per_step / 1e3) / 1e9
    points = {}
    for b, rec in recs.items():
        if b != args.batch and rec["decode_ms"][W:]:
            d = rec["decode_ms"][W:]
            points[f"decode_b{b}"] = round(b / (sum(d) / len(d) / 1e3), 1)
    prefill = None
    one = recs.get(1, main_rec)["prefill_steps"]
    whole = [(n, t) for n, n_dec, t in one if n == args.context and n_dec == 0]
    if whole:
        n, t = whole[0]
        prefill = {"value": round(n / (t / 1e3), 1), "tokens": n, "ms": round(t, 3),
                   "frac": round(prefill_flops(cfgd, args.layers, n) / (t / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    V = cfgd["vocab_size"]
    print(json.dumps({
        "metric": "decode tok/s at batch 8 (3B, bf16); prefill tok/s at 2,048 tokens and batch 1/64 beside it",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic: random weights N(0,0.02) in a GGUF file, random prompt characters",
        "config": {"model": "Qwen2.5-3B shape", "layers": args.layers, "layers_full": SHAPE_3B["num_hidden_layers"],
                   "global_batch": args.batch, "seq_len": args.context, "new_tokens": ra.NEW_TOKENS, "page": 16,
                   "parallelism": "single GPU", "program": "gpu_decoder_main, unmodified, nvcc -O3 -arch=sm_100",
                   "timing": "the program's own per-step wall-clock lines: batch building, copies, forward, "
                             "logits to the host and sampling there", "peaks": pk_src},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * 5 * args.batch,
                "d2h_bytes_per_step": 4 * V * args.batch, "ms_per_step": round(ms_per_step, 4)},
        "total_line": {"tokens": main_rec.get("total_tokens"), "seconds": main_rec.get("total_s")},
        "clocks": ck, "impl": "reference"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--shape", default="3B", choices=sorted(SHAPES), help="layer sizes: Qwen2.5-3B (the headline), 7B or 32B")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (config names both numbers)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--page-size", type=int, default=16, help="tokens in a page of the cache (a multiple of 16)")
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--timeline", action="store_true",
                    help="with --micro prefill_attention: print the kernel's own time stamps of one CTA (microseconds) to stderr")
    ap.add_argument("--micro", default=None, choices=["gemm", "decode_attention", "decode_attention_rope", "prefill_attention", "serve", "mixed_step"],
                    help="time one kernel alone at the 3B shape (for profiles/), or with 'serve' a whole run of "
                         "--batch requests (--context prompt tokens, --steps new tokens each) through the entry "
                         "point; print one JSON line and exit")
    ap.add_argument("--prefill-budget", type=int, default=512, help="serve: prompt tokens per step")
    ap.add_argument("--context-range", default=None, metavar="A:B", help="serve: prompt lengths uniform in [A, B]")
    ap.add_argument("--points", default="1,64", help="other decode batch sizes measured beside --batch")
    ap.add_argument("--micro-impl", default="stream", choices=["stream", "regs", "tc5", "cublas"])
    ap.add_argument("--micro-shape", default="lm_head", choices=["qkv", "o", "gate_up", "down", "lm_head"])
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--micro-graph", action="store_true", help="gemm: time inside a replayed graph, cold weights")
    ap.add_argument("--micro-splits", type=int, default=1, help="gemm with --micro-graph: shares of K (partial sums)")
    ap.add_argument("--history", type=int, default=2048, help="mixed_step: cached tokens before the prompt portion")
    ap.add_argument("--stamps", action="store_true",
                    help="for profiles/: run the decode step (up to 8 requests) with the attention and feed-forward "
                         "kernels writing their own time stamps, and print where a launch of each spends its time")
    ap.add_argument("--without", default=None, metavar="KINDS",
                    help="for profiles/: time the decode step with the kernels of these kinds left out (comma list of "
                         "ffn, attention, projections, norms for up to 8 requests; attention, products, norms, rope, swiglu "
                         "for more than 16); the step's results are void, only its time is printed")
    args = ap.parse_args()
    shape = SHAPES[args.shape]
    if args.layers is None:
        args.layers = shape["num_hidden_layers"]
    if args.micro:
        return micro(args)
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    W = max(3, args.warmup)
    K = max(1, args.steps)

    import torch
    from qwen_decoder_b200 import kernels
    from qwen_decoder_b200.config import Qwen2Config
    from qwen_decoder_b200.engine import Engine, SamplingParams, StepEntry
    from qwen_decoder_b200.parts import matmul_backend

    cfgd = dict(shape, num_hidden_layers=args.layers)
    cfg = Qwen2Config.from_dict(cfgd)
    pk, pk_src = peaks()
    page = args.page_size
    point_batches = [int(b) for b in args.points.split(",") if b] if not args.no_points else []
    max_b = max([args.batch] + point_batches)
    span = args.context + 2 * (W + K) + 64
    num_pages = max(max_b * ((span + page - 1) // page), (args.prefill_tokens + page - 1) // page) + 64
    torch.manual_seed(0)
    engine = Engine(config=cfg, random_seed=0, dtype="bfloat16", device="cuda:0", max_batch=max_b,
                    max_prefill_len=1 << 20, max_prefill_tokens_per_step=4096, max_total_tokens=8192,
                    page_size=page, num_pages=num_pages, max_positions=max(span, args.prefill_tokens) + 4096)
    runner = engine.runner
    dev = runner.device
    for kv in runner.cache.kv:                       # random cache contents stand in for real prompts
        kv.normal_(0.0, 1.0)
    gen = torch.Generator().manual_seed(1)

    def open_requests(n, tag):
        rcs = []
        for i in range(n):
            rc = runner.open(f"{tag}{i}")
            runner.cache.ensure(rc, args.context)
            runner.cache.commit(rc, args.context)
            rcs.append(rc)
        return rcs

    def time_decode(batch, steps, warm):
        rcs = open_requests(batch, f"b{batch}_")
        toks = torch.randint(0, cfg.vocab_size, (warm + steps, batch), generator=gen).tolist()
        zeros = ([0.0] * batch, [0] * batch, [0.0] * batch)
        for i in range(warm):
            runner.step([StepEntry(rc, [toks[i][j]], [0]) for j, rc in enumerate(rcs)], sampling=zeros)
        torch.cuda.synchronize(dev)
        l0 = kernels.launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warm, warm + steps):
            runner.step([StepEntry(rc, [toks[i][j]], [0]) for j, rc in enumerate(rcs)], sampling=zeros)
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1)
        launches = kernels.launches() - l0
        ctx_mean = args.context + warm + steps / 2.0
        for rc in rcs:
            runner.close(rc)
        return ms, launches, ctx_mean

    if args.stamps:
        # The kernels' own nanosecond stamps (%globaltimer) inside real, replayed steps: the buffers belong to the last
        # layer's launches of the last step.  Medians over the CTAs, microseconds from the first CTA's start.
        tl_a = torch.zeros(1024 * 16, dtype=torch.int64, device=dev)
        tl_f = torch.zeros(1024 * 8, dtype=torch.int64, device=dev)
        attn, ffn = kernels.decode_attention_rope, kernels.ffn_stream
        kernels.decode_attention_rope = lambda *a, **k: attn(*a, timeline=tl_a, **k)
        kernels.ffn_stream = lambda x, wgu, wd, barrier: ffn(x, wgu, wd, barrier, timeline=tl_f)
        ms, _, _ = time_decode(args.batch, K, W)
        torch.cuda.synchronize(dev)

        def table(tl, width, names):
            rows = [r for r in tl.view(-1, width).cpu().tolist() if r[0] > 0]
            if not rows:
                return ["  (this kernel did not run in the step)"]
            t0 = min(r[0] for r in rows)
            out = [f"  {len(rows)} CTAs"]
            for i, name in enumerate(names):
                v = sorted((r[i] - t0) / 1e3 for r in rows if r[i] > r[0] or i == 0)
                if v:
                    out.append(f"  {name:34s} min {v[0]:6.2f}  median {v[len(v) // 2]:6.2f}  max {v[-1]:6.2f}  (n={len(v)})")
            return out
        print(f"decode step, batch {args.batch}, context {args.context}: {ms / K:.4f} ms a step", file=sys.stderr)
        print("decode attention from partial sums:", file=sys.stderr)
        print("\n".join(table(tl_a, 16, ["start", "first chunks of keys asked for", "kernel before it done", "q built",
                                         "keys done", "warps merged, partial sums written", "ticket taken",
                                         "splits combined (one CTA per token and KV head)"])), file=sys.stderr)
        print("feed-forward in one launch:", file=sys.stderr)
        print("\n".join(table(tl_f, 8, ["start", "tokens there", "first tile written", "first product done",
                                        "its columns of h counted", "h there", "second product done"])), file=sys.stderr)
        return 0
    if args.without:
        # What does each kind of kernel add to the step?  Their launchers are replaced by nothing (outputs keep
        # whatever they held), the step is captured and replayed as usual, and only the time is reported.
        kinds = [k for k in args.without.split(",") if k]
        unknown = set(kinds) - {"ffn", "attention", "projections", "norms", "products", "rope", "swiglu"}
        if unknown:
            print(f"bench.py: --without takes ffn, attention, projections, norms, products, rope, swiglu; not {sorted(unknown)}")
            return 2
        held = {}

        def buffer(shape, dtype):
            return held.setdefault((tuple(shape), dtype), torch.zeros(shape, dtype=dtype, device=dev))
        if "ffn" in kinds:
            kernels.ffn_stream = lambda x, wgu, wd, barrier: buffer(
                (kernels.skinny_splits(x.shape[1], wd.shape[1], x.shape[0]), x.shape[0], x.shape[1]), torch.float32)
        if "attention" in kinds:
            kernels.decode_attention_rope = lambda *a, **k: None
            kernels.decode_attention = lambda *a, **k: None
        if "products" in kinds:                    # the library products of more than 16 tokens
            matmul_backend._cublas = lambda x, w, bias, out: None
        if "rope" in kinds:
            kernels.rope_kv_write = lambda *a, **k: None
        if "swiglu" in kinds:
            kernels.swiglu = lambda *a, **k: None
        if "projections" in kinds:
            kernels.gemm_skinny_partial = lambda x, w, splits: buffer((splits, x.shape[0], w.shape[0]), torch.float32)
        if "norms" in kinds:
            kernels.add_rmsnorm = lambda *a, **k: None
        ms, launches, _ = time_decode(args.batch, K, W)
        print(json.dumps({"micro": "decode_step_without", "without": kinds, "batch": args.batch, "context": args.context,
                          "layers": args.layers, "steps": K, "ms_per_step": round(ms / K, 4), "launches_per_step": launches // K,
                          "note": "the step's results are void: a measurement of what each kind of kernel adds"}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    ms, launches, ctx_mean = time_decode(args.batch, K, W)
    value = args.batch * K / (ms / 1e3)
    ms_per_step = ms / K
    bytes_step = decode_bytes(cfgd, args.layers, args.batch, ctx_mean)
    achieved = bytes_step / (ms_per_step / 1e3) / 1e9

    points = {}
    if not args.no_points:
        for b in point_batches:
            if b == args.batch:
                continue
            pms, _, _ = time_decode(b, min(K, 128), W)
            points[f"decode_b{b}"] = round(b * min(K, 128) / (pms / 1e3), 1)

    # prefill: one prompt of T tokens in one step, logits at its last place; the events span the host's
    # launching too, so a portion that the host cannot launch as fast as the device runs it shows here
    def time_prefill(T, tag):
        pre_ms = []
        for i in range(W + 3):
            rc = runner.open(f"{tag}{i}")
            prompt = torch.randint(0, cfg.vocab_size, (T,), generator=gen).tolist()
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step([StepEntry(rc, prompt, [T - 1])])
            e1.record()
            torch.cuda.synchronize(dev)
            if i >= W:
                pre_ms.append(e0.elapsed_time(e1))
            runner.close(rc)
        return sorted(pre_ms)[len(pre_ms) // 2]

    T = args.prefill_tokens
    pre = time_prefill(T, "p")
    if not args.no_points:
        for t in (128, 512):
            points[f"prefill_{t}"] = round(t / (time_prefill(t, f"q{t}_") / 1e3), 1)
    pflops = prefill_flops(cfgd, args.layers, T)
    prefill = {"value": round(T / (pre / 1e3), 1), "tokens": T, "ms": round(pre, 3),
               "frac": round(pflops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # end to end through the entry point: host ids in, sampled ids out, every step
    e2e = None
    if not args.no_e2e:
        sp = SamplingParams(max_new_tokens=W + K + 8, ignore_eos=True)
        reqs = []
        for i in range(args.batch):
            r = engine.add_request(torch.randint(0, cfg.vocab_size, (64,), generator=gen).tolist(), sp)
            reqs.append(r)
        while any(r.num_pending > 1 or not r.output for r in reqs):
            engine.step()
        # lengthen every request's cache to the benchmark context without running long prompts
        for r in reqs:
            add = args.context - r.cache.num_tokens
            runner.cache.ensure(r.cache, r.cache.num_tokens + add)
            runner.cache.commit(r.cache, add)
            r.num_computed += add
            r.prompt = r.prompt + [0] * add
        for _ in range(W):
            engine.step()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        n0 = sum(len(r.output) for r in reqs)
        for _ in range(K):
            engine.step()
        e1.record()
        torch.cuda.synchronize(dev)
        wall = time.perf_counter() - t0
        n1 = sum(len(r.output) for r in reqs)
        bp = 1
        while bp < args.batch:
            bp *= 2
        # the packed metadata of this batch size's graphs (other sizes' graphs, made for ``points``, are larger)
        h2d = max((gr.lay.total * 4 for gr in runner._graphs.values() if gr.lay.T == bp), default=0)
        e2e = {"value": round((n1 - n0) / max(wall, e0.elapsed_time(e1) / 1e3), 1), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch, "ms_per_step": round(wall / K * 1e3, 4)}
    ck = clocks.stop()

    out = {
        "metric": f"decode tok/s at batch {args.batch} ({args.shape}, bf16); prefill tok/s at {args.prefill_tokens:,} tokens and "
                  "batch 1/64 beside it",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), random token ids, random cache contents",
        "config": {"model": f"Qwen2.5-{args.shape} shape", "layers": args.layers, "layers_full": shape["num_hidden_layers"],
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": bool(cfgd["tie_word_embeddings"]), "global_batch": args.batch, "seq_len": args.context, "new_tokens": W + K,
                   "page": page, "parallelism": "single GPU", "l2": f"inputs larger than L2 (weights {decode_bytes(cfgd, args.layers, 0, 0) / 1e9:.1f} GB/step)",
                   "bf16_gemm": matmul_backend.mode, "peaks": pk_src},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "e2e": e2e, "gpu_launches": launches, "library_gemms": matmul_backend.counters["library"],
        "clocks": ck, "impl": "ours",
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
