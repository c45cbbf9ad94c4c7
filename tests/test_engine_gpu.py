"""The engine against the plain implementation, in float32 and in bfloat16, for every way
of cutting the work: whole, decoded tail, changing portions, mixed with page reuse."""
import random

import numpy as np
import pytest
import torch

import plain_model
import trace_tools
from tiny_configs import TINY, make_folder

pytestmark = pytest.mark.gpu

# max |logit difference| relative to the largest |logit|, fixed in advance:
# float32 differs from the float64 plain implementation by rounding of sums only;
# bfloat16 rounds every activation to 8 bits of mantissa over a few layers.
TOL = {"float32": 1e-5, "bfloat16": 3e-2}
LENGTHS = {"A": [5, 17, 33, 70, 150], "B": [1, 9, 64, 130, 200], "C": [3, 40, 97, 180], "D": [2, 66, 129, 300, 515]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in TINY:
        folder = make_folder(name, str(tmp_path_factory.mktemp(f"tiny{name}")))
        cfg, w = plain_model.read_folder(folder)
        rng = random.Random(100 + ord(name))
        seqs = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in LENGTHS[name]]
        want = [plain_model.forward(cfg, w, s).numpy() for s in seqs]
        out[name] = (folder, cfg, w, seqs, want)
    return out


def make_runner(folder, dtype, max_tokens, page_size=16):
    from qwen_decoder_b200.engine import ModelRunner
    return ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0",
                                   num_pages=(max_tokens + page_size - 1) // page_size,
                                   page_size=page_size, max_requests=8)


def held(seqs):
    return max((len(s) + 63) // 64 * 64 for s in seqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name]
    runner = make_runner(folder, dtype, held(seqs), page_size=32 if name == "B" else 16)
    tr = trace_tools.whole(seqs)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want, TOL[dtype])
    runner.cache.check()
    assert runner.cache.free_pages() == [runner.cache.num_pages] * len(runner.cache.pools)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_decode_tail(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name]
    runner = make_runner(folder, dtype, held(seqs))
    tr = trace_tools.decode_tail(seqs, tail=32)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name]
    runner = make_runner(folder, dtype, held(seqs), page_size=32 if name == "B" else 16)
    tr = trace_tools.portions(seqs)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_with_page_reuse(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name]
    # twice every request, in two orders, in a pool that holds about two of the longest
    seqs2 = seqs + seqs[::-1]
    want2 = want + want[::-1]
    max_tokens = 2 * held(seqs)
    runner = make_runner(folder, dtype, max_tokens)
    tr = trace_tools.mixed(seqs2, max_tokens, seed=7)
    assert sum(len(s["entries"]) > 1 for s in tr.steps) > 5
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want2, TOL[dtype])
    runner.cache.check()
    assert runner.cache.free_pages() == [runner.cache.num_pages] * len(runner.cache.pools)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_does_not_change_float32_logits(models, dtype, tmp_path):
    """Between two ways of cutting, logits agree far more closely than with the plain implementation."""
    folder, cfg, w, seqs, want = models["A"]
    r1 = make_runner(folder, dtype, held(seqs))
    a = trace_tools.whole(seqs)
    ga = trace_tools.run_inprocess(r1, a, str(tmp_path / "a"))
    b = trace_tools.portions(seqs)
    gb = trace_tools.run_inprocess(r1, b, str(tmp_path / "b"))
    rows_a = {rp: ga[s][i] for s, rows in a.expect.items() for i, rp in enumerate(rows)}
    rows_b = {rp: gb[s][i] for s, rows in b.expect.items() for i, rp in enumerate(rows)}
    scale = max(float(np.abs(x).max()) for x in want)
    worst = max(float(np.abs(rows_a[k] - rows_b[k]).max()) for k in rows_a)
    assert worst <= (1e-6 if dtype == "float32" else TOL[dtype]) * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(models, dtype, tmp_path):
    """A prompt of 3 tokens and then 250 tokens one by one (crossing many pages); the first
    positions of a sequence are compared one by one as well."""
    folder, cfg, w, seqs, want = models["A"]
    rng = random.Random(5)
    seq = [rng.randrange(cfg["vocab_size"]) for _ in range(253)]
    expect = [plain_model.forward(cfg, w, seq).numpy()]
    runner = make_runner(folder, dtype, 256)
    tr = trace_tools.decode_tail([seq], tail=250)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, expect, TOL[dtype])


def test_float16_weights_are_exact_in_float32_and_rounded_once_in_bfloat16(tmp_path):
    """A folder stored in float16, the reference's own weight format (common.cpp:104-112), which its
    float32 forward decodes exactly (cpu_decoder.cpp:55-62): the float32 engine must use every stored
    bit, the bfloat16 engine rounds each weight once."""
    from qwen_decoder_b200.config import Qwen2Config
    from qwen_decoder_b200.weights import write_random_model
    folder = write_random_model(Qwen2Config.from_dict(TINY["A"]), str(tmp_path / "f16"), 5, dtype=torch.float16)
    cfg, w = plain_model.read_folder(folder)
    assert any((t.float().bfloat16().double() != t).any() for t in w.values())     # bits that bfloat16 would lose
    rng = random.Random(9)
    seqs = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (9, 60)]
    want = [plain_model.forward(cfg, w, s).numpy() for s in seqs]
    for dtype in ("float32", "bfloat16"):
        runner = make_runner(folder, dtype, held(seqs))
        tr = trace_tools.portions(seqs)
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / dtype))
        trace_tools.compare(tr, got, want, TOL[dtype])
