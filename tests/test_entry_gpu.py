"""Generation through the Python entry point and the command line, and the replay program as a
user runs it."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model
import trace_tools
from tiny_configs import TINY, make_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(n, str(tmp_path_factory.mktemp(f"m{n}"))) for n in ("A", "B")}


def prompts_for(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]


def check_greedy(cfg, w, prompt, got, dtype):
    """Greedy tokens equal the plain implementation's, up to the first near tie of its logits."""
    want, margins = plain_model.greedy_generate(cfg, w, prompt, len(got))
    limit = 1e-4 if dtype == "float32" else 2e-2
    n = next((i for i, m in enumerate(margins) if m < limit), len(want))
    assert got[:n] == want[:n], (prompt, got, want, margins)
    return n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folders, dtype):
    """Tiny A's workload: prompts of 5, 17 and 33 ids, 16 greedy tokens each."""
    from qwen_decoder_b200.engine import Engine, SamplingParams
    cfg, w = plain_model.read_folder(folders["A"])
    prompts = prompts_for(cfg, [5, 17, 33], seed=0)
    eng = Engine(folders["A"], dtype=dtype, num_pages=32, max_batch=4)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=16))
    assert all(len(o) == 16 for o in outs)
    checked = sum(check_greedy(cfg, w, p, o, dtype) for p, o in zip(prompts, outs))
    assert checked >= 24
    assert eng.runner.cache.free_pages() == [32]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_chunked_prefill_mixed_with_decode_and_temperature(folders, dtype):
    """Tiny B's workload: prompts of 1, 9, 64 and 130 ids in 24-token portions mixed with decode tokens,
    20 tokens at temperature 0.8 with a fixed sampler seed.  The same request gives the same tokens
    alone and in the batch, and in a pool so small that requests are preempted."""
    from qwen_decoder_b200.engine import Engine, SamplingParams
    cfg, w = plain_model.read_folder(folders["B"])
    prompts = prompts_for(cfg, [1, 9, 64, 130], seed=1)
    sp = SamplingParams(temperature=0.8, max_new_tokens=20, seed=123)
    eng = Engine(folders["B"], dtype=dtype, num_pages=16, page_size=32, max_batch=4, max_prefill_tokens_per_step=24)
    outs = eng.generate(prompts, sp)
    assert all(len(o) == 20 for o in outs) and eng.stats["prompt_tokens"] == 204
    assert len({tuple(o) for o in outs}) == 4
    if dtype == "bfloat16":
        # with a thousand nearly equal probabilities, bfloat16 rounding of the logits moves the running sum
        # by more than the distance between its steps, so single tokens cannot be pinned against the plain
        # implementation here; float32 pins the sampling path, bfloat16 must at least repeat itself
        again = Engine(folders["B"], dtype=dtype, num_pages=16, page_size=32, max_batch=4,
                       max_prefill_tokens_per_step=24)
        assert again.generate(prompts, sp) == outs
        return
    # each token is what the plain sampler draws from the plain logits with the same uniform draw
    from qwen_decoder_b200.sampling import uniform_draw
    checked = 0
    for i, (p, o) in enumerate(zip(prompts, outs)):
        seq = list(p)
        for j, tok in enumerate(o):
            logits = plain_model.forward(cfg, w, seq)[-1]
            want, margin = plain_model.sample_topk(logits, 0, 0.8, uniform_draw(123, i, j))
            seq.append(tok)        # go on along the engine's own tokens
            if margin < 1e-5:
                continue           # float32 rounding of the running sum could decide this draw either way
            assert tok == want, (i, j, tok, want)
            checked += 1
    assert checked >= 60
    # alone, one request at a time, nothing cut: same tokens (draws are keyed by request, not by batch)
    for i, p in enumerate(prompts):
        solo = Engine(folders["B"], dtype=dtype, num_pages=16, page_size=32)
        solo._next_id = i
        assert solo.generate([p], sp)[0] == outs[i]
    # a pool of 5 pages of 32 tokens: the longest request is admitted beside another, outgrows the pool,
    # is preempted and recomputed later -- with the same tokens
    small = Engine(folders["B"], dtype=dtype, num_pages=5, page_size=32, max_batch=4,
                   max_prefill_tokens_per_step=24)
    assert small.generate(prompts, sp) == outs
    assert small.stats["preemptions"] >= 1 and small.runner.cache.free_pages() == [5]


def test_command_line(folders):
    cfg, w = plain_model.read_folder(folders["A"])
    prompts = prompts_for(cfg, [4, 11], seed=2)
    stdin = "".join(" ".join(map(str, p)) + "\n" for p in prompts) + "\n"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "decoder_main"), folders["A"], "8", "4096", "16",
                        "64", "0", "--dtype", "float32", "--max-new-tokens", "6", "--num-pages", "16"],
                       input=stdin, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.startswith("[")]
    assert len(lines) == 2 and "tokens/s" in r.stderr
    for p, line in zip(prompts, lines):
        got = [int(t) for t in line.split(")", 1)[1].split()]
        assert len(got) == 6 and check_greedy(cfg, w, p, got, "float32") >= 4


def test_command_line_options_beyond_the_reference(folders, tmp_path):
    """--random-weights on a folder with config.json only, prompts from --prompt-ids, a file and --random-prompts,
    --stats: a line per step in the reference's words, and prompt / decode tokens per second apart."""
    import json
    import shutil
    only_config = tmp_path / "cfg"
    only_config.mkdir()
    shutil.copy(os.path.join(folders["A"], "config.json"), only_config / "config.json")
    pf = tmp_path / "prompts.txt"
    pf.write_text("5 6 7 8 9\n10,11,12\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "decoder_main"), str(only_config), "4", "4096", "8",
                        "64", "0", "--random-weights", "--weights-seed", "3", "--prompt-ids", "1,2,3", "--prompt-file",
                        str(pf), "--random-prompts", "2", "--len", "3:20", "--max-new-tokens", "5", "--num-pages", "24",
                        "--ignore-eos", "--stats"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.startswith("[")]
    assert len(lines) == 5 and all(len(l.split(")", 1)[1].split()) == 5 for l in lines)
    steps = [l for l in r.stderr.splitlines() if l.startswith("step ")]
    assert steps and all("total_tokens=" in l and "n_decode=" in l and "prefill_tokens=" in l and "ms=" in l for l in steps)
    # prompts are cut under the budget of 8 prompt tokens a step
    assert all(int(l.split("prefill_tokens=")[1].split()[0]) <= 8 for l in steps)
    assert any(l.startswith("prompt: ") and "decode: " in l and "tokens/s" in l for l in r.stderr.splitlines())
    # the same seed gives the same weights: the same tokens again
    r2 = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "decoder_main"), str(only_config), "4", "4096", "64",
                         "64", "0", "--random-weights", "--weights-seed", "3", "--prompt-ids", "1,2,3",
                         "--max-new-tokens", "5", "--num-pages", "24", "--ignore-eos"], capture_output=True, text=True,
                        timeout=600)
    assert r2.returncode == 0, r2.stderr
    assert [l for l in r2.stdout.splitlines() if l.startswith("[")][0] == lines[0]


def test_step_records(folders):
    from qwen_decoder_b200.engine import Engine, SamplingParams
    cfg, _ = plain_model.read_folder(folders["A"])
    eng = Engine(folders["A"], dtype="bfloat16", num_pages=32, max_prefill_tokens_per_step=16, record_steps=True)
    prompts = prompts_for(cfg, [40, 5, 23], seed=8)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    recs = eng.step_records()
    assert sum(r["prompt_tokens"] for r in recs) == 68 and sum(r["decode_tokens"] for r in recs) == 3 * 5
    assert all(r["prompt_tokens"] <= 16 and r["ms"] > 0 and r["tokens"] == r["prompt_tokens"] + r["decode_tokens"]
               for r in recs)
    assert any(r["planned_ahead"] for r in recs) and recs[-1]["pages_free"][0] < 32
    assert [len(o) for o in outs] == [6, 6, 6]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program_with_pages_of_32(folders, dtype, tmp_path):
    """Tiny B's page of 32 tokens through the program itself (--page-size), four requests live at most."""
    cfg, w = plain_model.read_folder(folders["B"])
    seqs = prompts_for(cfg, [1, 9, 64, 130, 70], seed=4)
    want = [plain_model.forward(cfg, w, s).numpy() for s in seqs]
    tr = trace_tools.mixed(seqs, max_tokens=320, seed=2)
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"], "--dtype",
                        dtype, "--out", str(out), "--max-tokens", "320", "--page-size", "32", "--max-live", "4"],
                       input=tr.lines(), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    assert r.stdout.splitlines() == [f"done {s['step']}" for s in tr.steps]
    got = trace_tools.read_outputs(tr, str(out), cfg["vocab_size"])
    trace_tools.compare(tr, got, want, 1e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folders, dtype, tmp_path):
    """bin/trace_run as a separate process: steps on stdin, one `done` line per step, .f32 files."""
    cfg, w = plain_model.read_folder(folders["B"])
    seqs = prompts_for(cfg, [40, 75, 20, 64, 33], seed=3)
    want = [plain_model.forward(cfg, w, s).numpy() for s in seqs]
    tr = trace_tools.mixed(seqs, max_tokens=256, seed=9)
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"], "--dtype",
                        dtype, "--out", str(out), "--max-tokens", "256"], input=tr.lines(), capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    assert r.stdout.splitlines() == [f"done {s['step']}" for s in tr.steps]
    got = trace_tools.read_outputs(tr, str(out), cfg["vocab_size"])
    trace_tools.compare(tr, got, want, 1e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefix_cache_shares_pages_and_keeps_logits(folders, dtype, tmp_path):
    """Requests with a common beginning: with the prefix cache the later ones skip the shared full pages,
    their logits still equal the plain implementation's, and generation gives the same tokens."""
    from qwen_decoder_b200.engine import Engine, ModelRunner, SamplingParams, StepEntry
    cfg, w = plain_model.read_folder(folders["A"])
    stem = prompts_for(cfg, [70], seed=5)[0]
    tails = prompts_for(cfg, [9, 3, 20], seed=6)
    seqs = [stem + t for t in tails]
    want = [plain_model.forward(cfg, w, s).numpy() for s in seqs]
    runner = ModelRunner.from_folder(folders["A"], dtype=dtype, device="cuda:0", num_pages=24, page_size=16,
                                     max_requests=4, prefix_cache=True)
    tol = 1e-5 if dtype == "float32" else 3e-2
    scale = max(float(np.abs(x).max()) for x in want)
    skipped = []
    live = []
    for i, s in enumerate(seqs):
        rc = runner.open(f"r{i}", s)
        start = rc.num_tokens
        skipped.append(start)
        rest = s[start:]
        logits = runner.step([StepEntry(rc, rest, list(range(len(rest))))]).cpu().numpy()
        err = float(np.abs(logits - want[i][start:]).max())
        assert err <= tol * scale, (i, err)
        live.append(rc)
        if i == 1:
            runner.close(live.pop(0))            # the first request ends; its pages stay cached
    assert skipped == [0, 64, 64]                # four full pages of the 70-token stem are shared
    runner.cache.check()
    for rc in live:
        runner.close(rc)
    assert runner.cache.free_pages() == [24]
    # through the entry point: same tokens with and without the cache, fewer prompt tokens computed
    sp = SamplingParams(max_new_tokens=6)
    outs = {}
    for on in (False, True):
        eng = Engine(folders["A"], dtype=dtype, num_pages=40, max_batch=2, enable_prefix_cache=on)
        outs[on] = (eng.generate(seqs, sp), eng.stats)
    assert outs[False][0] == outs[True][0]
    assert outs[True][1]["prompt_tokens"] < outs[False][1]["prompt_tokens"]
    assert outs[True][1].get("prefix_hit_tokens", 0) >= 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_changes_no_token(folders, dtype):
    """With ``run_ahead`` a decode step is launched before the tokens of the step before it are read:
    the outputs must equal those of the step-by-step engine -- greedy and with temperature, with stop
    tokens that end requests one step late for the device, with the prefix cache recording generated
    tokens -- and most decode steps must indeed have run ahead."""
    from qwen_decoder_b200.engine import Engine, SamplingParams
    cfg, _ = plain_model.read_folder(folders["A"])
    prompts = prompts_for(cfg, [5, 17, 33, 8], seed=3)

    def run(run_ahead):
        eng = Engine(folders["A"], dtype=dtype, num_pages=64, max_batch=4, run_ahead=run_ahead,
                     enable_prefix_cache=True)
        probe = eng.generate(prompts[:1], SamplingParams(max_new_tokens=12))[0]
        params = [SamplingParams(max_new_tokens=40, stop_ids=[probe[7]]),          # ends on a stop token
                  SamplingParams(max_new_tokens=25, temperature=0.7, seed=5, ignore_eos=True),
                  SamplingParams(max_new_tokens=31, ignore_eos=True),
                  SamplingParams(max_new_tokens=18, temperature=1.1, top_k=20, seed=9, ignore_eos=True)]
        # all requests are there from the start, so that both engines run the same batches (a request
        # that arrives in between is planned one step later when running ahead, and other batches round
        # the logits differently)
        reqs = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
        while eng.has_work():
            eng.step()
        assert eng.runner.cache.free_pages() == [64]
        eng.runner.cache.check()
        # the same prompt again: its pages, generated tokens included, are known to the prefix cache
        again = eng.generate([prompts[2] + reqs[2].output[:20]], SamplingParams(max_new_tokens=4, ignore_eos=True))
        return [r.output for r in reqs] + again, [r.finish_reason for r in reqs], eng.stats

    out_a, why_a, stats_a = run(True)
    out_b, why_b, stats_b = run(False)
    assert out_a == out_b and why_a == why_b
    assert why_a[0] == "stop" and len(out_a[0]) < 40
    assert stats_a["prefix_hit_tokens"] == stats_b["prefix_hit_tokens"] > 0
    assert stats_a["model_steps"] >= stats_b["model_steps"]      # a wasted row now and then, never fewer steps
