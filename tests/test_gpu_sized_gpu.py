"""The engine against the plain implementation at the layer sizes that serving and the benchmark run:
two-layer models with the sizes of Qwen2.5-3B (hidden 2048, 16 heads in 2 groups, head size 128,
intermediate 11008, vocabulary 151,936, tied) and of Qwen2.5-7B (hidden 3584, 28 heads in 4 groups of 7,
intermediate 18944, vocabulary 152,064, output matrix of its own), in float32 and bfloat16, cut every way,
with one sequence that crosses 2,048 positions (block tables of more than 128 pages, more than 8 shares
of the keys in decode attention); and decode steps of 13 to 64 requests at once, the batch sizes whose
kernels differ from those of small batches.

Weights are made on the device and handed to the engine and to the plain implementation (float64, on
the device too: tests/plain_model.py computes where its weights lie) without a folder in between.
Logits are compared at chosen positions, since a row of this vocabulary is 0.6 MB.
"""
import random

import numpy as np
import pytest
import torch

import plain_model
import trace_tools
from tiny_configs import TINY

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 1e-5, "bfloat16": 3e-2}

SHAPES = {
    "3B": dict(architectures=["Qwen2ForCausalLM"], hidden_size=2048, intermediate_size=11008, num_hidden_layers=2,
               num_attention_heads=16, num_key_value_heads=2, vocab_size=151936, max_position_embeddings=4096,
               rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "7B": dict(architectures=["Qwen2ForCausalLM"], hidden_size=3584, intermediate_size=18944, num_hidden_layers=2,
               num_attention_heads=28, num_key_value_heads=4, vocab_size=152064, max_position_embeddings=4096,
               rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False),
}
LENGTHS = [37, 300, 2100]
PROMPT_FRAC = 0.97          # in the mixed trace: the rest of a request is fed token by token


def keep(n):
    """Positions of a sequence of n tokens whose logits the traces ask for: the first, the last 34, every
    61st, and both sides of every 512th (page edges and the edges of the kernels' key tiles)."""
    return lambda p: p < 3 or p >= n - 34 or p % 61 == 0 or p % 512 in (0, 511)


class Big:
    """A model's tensors (bfloat16, on the device), its plain float64 twin, sequences and expected rows."""

    def __init__(self, name):
        from qwen_decoder_b200.config import Qwen2Config, describe_model
        from qwen_decoder_b200.parts.model import build_model
        from qwen_decoder_b200.weights.random_init import random_tensors
        self.cfg_dict = SHAPES[name]
        self.config = Qwen2Config.from_dict(self.cfg_dict)
        specs = build_model(describe_model(self.config)).tensor_specs()
        self.tensors = random_tensors(specs, seed=40 + len(name), dtype=torch.bfloat16, device=DEV)
        w64 = {n: t.double() for n, t in self.tensors.items()}
        rng = random.Random(7)
        V = self.cfg_dict["vocab_size"]
        self.seqs = [[rng.randrange(V) for _ in range(n)] for n in LENGTHS]
        self.want = []
        for seq in self.seqs:
            n = len(seq)
            k = keep(n)
            rows = sorted({p for p in range(n) if k(p)} | set(range(int(n * PROMPT_FRAC) - 1, n)))
            logits = plain_model.forward(self.cfg_dict, w64, seq, rows=rows).float().cpu().numpy()
            self.want.append({p: logits[i] for i, p in enumerate(rows)})
        self.w64 = w64

    def keep(self, r, p):
        return keep(len(self.seqs[r % len(self.seqs)]))(p)

    def runner(self, dtype, max_tokens, **kw):
        from qwen_decoder_b200.config import describe_model
        from qwen_decoder_b200.engine import ModelRunner
        from qwen_decoder_b200.engine.runner import resolve_dtype
        from qwen_decoder_b200.parts.model import build_model
        from qwen_decoder_b200.weights import TensorSource, load_into
        model = build_model(describe_model(self.config))
        load_into(model, TensorSource.from_dict(self.tensors), resolve_dtype(dtype), torch.device(DEV))
        kw.setdefault("max_requests", 8)
        return ModelRunner(model, self.config, num_pages=(max_tokens + 15) // 16, page_size=16, **kw)


@pytest.fixture(scope="module")
def big():
    made = {}

    def get(name):
        if name not in made:
            made.clear()                  # one model's float64 twin at a time
            torch.cuda.empty_cache()
            made[name] = Big(name)
        return made[name]
    yield get
    made.clear()
    torch.cuda.empty_cache()


def held(seqs):
    return max((len(s) + 63) // 64 * 64 for s in seqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["3B", "7B"])
def test_whole_and_decoded_tail(big, name, dtype, tmp_path):
    m = big(name)
    runner = m.runner(dtype, held(m.seqs))
    for i, tr in enumerate([trace_tools.whole(m.seqs, keep=m.keep), trace_tools.decode_tail(m.seqs, 32, keep=m.keep)]):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{i}"))
        trace_tools.compare(tr, got, m.want, TOL[dtype])
    runner.cache.check()
    assert runner.cache.free_pages() == [runner.cache.num_pages]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["3B", "7B"])
def test_portions_of_changing_size(big, name, dtype, tmp_path):
    m = big(name)
    runner = m.runner(dtype, held(m.seqs))
    # long portions too: a portion of 512 tokens over hundreds of cached ones is what serving runs
    tr = trace_tools.portions(m.seqs, sizes=(500, 2, 24, 130, 3, 512, 2, 16, 7), keep=m.keep)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, m.want, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["3B", "7B"])
def test_mixed_with_page_reuse(big, name, dtype, tmp_path):
    m = big(name)
    seqs2, want2 = m.seqs + m.seqs[::-1], m.want + m.want[::-1]
    max_tokens = held(m.seqs) + 512          # the two long requests never fit together: pages are used again
    runner = m.runner(dtype, max_tokens)
    keep2 = lambda r, p: keep(len(seqs2[r]))(p)
    tr = trace_tools.mixed(seqs2, max_tokens, seed=11, prompt_frac=PROMPT_FRAC, keep=keep2,
                           portion_sizes=(2, 5, 24, 130, 400))
    assert sum(len(s["entries"]) > 1 for s in tr.steps) > 5
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want2, TOL[dtype])
    runner.cache.check()
    assert runner.cache.free_pages() == [runner.cache.num_pages]


# ---------------------------------------------------------------- many requests decoding together
def _many_requests(cfg_dict, w64, n_req, longest, n_new, seed):
    """Sequences of different lengths (a few long ones), and the plain logits at their last n_new places."""
    rng = random.Random(seed)
    V = cfg_dict["vocab_size"]
    lens = [rng.randrange(3, longest // 4) for _ in range(n_req)]
    lens[1], lens[n_req // 2], lens[-1] = longest, longest * 2 // 3, longest // 2 + 5
    seqs = [[rng.randrange(V) for _ in range(n + n_new)] for n in lens]
    want = []
    for seq in seqs:
        rows = list(range(len(seq) - n_new - 1, len(seq)))
        logits = plain_model.forward(cfg_dict, w64, seq, rows=rows).float().cpu().numpy()
        want.append({p: logits[i] for i, p in enumerate(rows)})
    return lens, seqs, want


def _decode_together(runner, lens, seqs, want, n_new, dtype):
    """Prompts in steps of a few requests, then n_new steps of all requests' single tokens."""
    from qwen_decoder_b200.engine import StepEntry
    rcs = [runner.open(i) for i in range(len(seqs))]
    scale = max(float(np.abs(v).max()) for w in want for v in w.values())
    worst = 0.0

    def check(logits, places):
        nonlocal worst
        got = logits.float().cpu().numpy()
        for row, (r, p) in enumerate(places):
            err = float(np.abs(got[row] - want[r][p]).max())
            worst = max(worst, err)
            assert err <= TOL[dtype] * scale, f"request {r} (prompt {lens[r]}) position {p}: {err:.3e} of {scale:.3e}"

    for a in range(0, len(seqs), 6):
        group = list(range(a, min(a + 6, len(seqs))))
        logits = runner.step([StepEntry(rcs[r], seqs[r][:lens[r]], [lens[r] - 1]) for r in group])
        check(logits, [(r, lens[r] - 1) for r in group])
    for j in range(n_new):
        logits = runner.step([StepEntry(rcs[r], [seqs[r][lens[r] + j]], [0]) for r in range(len(seqs))])
        check(logits, [(r, lens[r] + j) for r in range(len(seqs))])
    for rc in rcs:
        runner.close(rc)
    runner.check_status()
    runner.cache.check()
    return worst / scale


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_req", [13, 24, 64])
def test_many_requests_decode_together_tiny(n_req, dtype, graphs, tmp_path):
    from tiny_configs import make_folder
    from qwen_decoder_b200.engine import ModelRunner
    folder = make_folder("D", str(tmp_path))
    cfg, w = plain_model.read_folder(folder)
    lens, seqs, want = _many_requests(cfg, w, n_req, longest=600, n_new=20, seed=n_req)
    pages = sum((len(s) + 15) // 16 for s in seqs) + 4
    runner = ModelRunner.from_folder(folder, dtype=dtype, device=DEV, num_pages=pages, page_size=16,
                                     max_requests=n_req, use_graphs=graphs)
    _decode_together(runner, lens, seqs, want, 20, dtype)
    assert bool(runner._graphs) == graphs


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_req", [16, 24, 64])
def test_many_requests_decode_together_3b_sizes(big, n_req, dtype, graphs):
    m = big("3B")
    lens, seqs, want = _many_requests(m.cfg_dict, m.w64, n_req, longest=2200, n_new=20, seed=100 + n_req)
    pages_tokens = sum((len(s) + 15) // 16 * 16 for s in seqs) + 64
    runner = m.runner(dtype, pages_tokens, max_requests=n_req, use_graphs=graphs)
    _decode_together(runner, lens, seqs, want, 20, dtype)
    assert bool(runner._graphs) == graphs


@pytest.mark.parametrize("n_req", [24, 64])
def test_running_ahead_and_graphs_do_not_change_the_tokens(n_req, tmp_path):
    """Greedy generation for many requests at once through the entry point: the same tokens with and without
    CUDA graphs and with and without running ahead, and the plain implementation's tokens up to the first
    place where its two best logits are nearly tied."""
    from tiny_configs import make_folder
    from qwen_decoder_b200.engine import Engine, SamplingParams
    folder = make_folder("B", str(tmp_path))       # an output matrix of its own: tokens do not repeat the input
    cfg, w = plain_model.read_folder(folder)
    rng = random.Random(n_req)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randrange(2, 90))] for _ in range(n_req)]
    outs = {}
    for graphs in (True, False):
        for ahead in (True, False):
            eng = Engine(folder, dtype="bfloat16", device=DEV, max_batch=n_req, num_pages=n_req * 8 + 8,
                         max_prefill_tokens_per_step=128, use_graphs=graphs, run_ahead=ahead)
            outs[(graphs, ahead)] = eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
            assert eng.runner.cache.free_pages() == [n_req * 8 + 8]
    first = outs[(True, True)]
    for key, o in outs.items():
        assert o == first, f"use_graphs, run_ahead = {key}: other tokens than with both on"
    checked = 0
    for prompt, out in list(zip(prompts, first))[:24]:
        plain, margins = plain_model.greedy_generate(cfg, w, prompt, 12)
        n = next((i for i, mg in enumerate(margins) if mg < 2e-2), len(plain))
        assert out[:n] == plain[:n]
        checked += n
    assert checked >= 20
