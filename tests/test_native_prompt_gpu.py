"""Prompt steps whose layers are launched from the native loop against the same steps launched part by
part, and against the plain implementation; and which models the native loop declines."""
import random

import numpy as np
import pytest
import torch

import plain_model
from tiny_configs import TINY, make_folder

pytestmark = pytest.mark.gpu


def runner_for(folder, native: bool):
    from qwen_decoder_b200.engine import ModelRunner
    r = ModelRunner.from_folder(folder, dtype="bfloat16", device="cuda:0", num_pages=64, page_size=16, max_requests=4)
    if not native:
        r.model.native_prompt = None
    return r


def run_portions(runner, seqs, cuts):
    """Each sequence in portions of ``cuts`` tokens, the sequences side by side in one step; logits of every
    portion's last token, keyed by (sequence, position)."""
    from qwen_decoder_b200.engine import StepEntry
    rcs = [runner.open(f"s{i}") for i in range(len(seqs))]
    done = [0] * len(seqs)
    out = {}
    for cut in cuts:
        entries, keys = [], []
        for i, s in enumerate(seqs):
            part = s[done[i]:done[i] + cut]
            if part:
                entries.append(StepEntry(rcs[i], part, [len(part) - 1]))
                done[i] += len(part)
                keys.append((i, done[i] - 1))
        if not entries:
            break
        logits = runner.step(entries).float().cpu().numpy()
        for k, row in zip(keys, logits):
            out[k] = row
    for rc in rcs:
        runner.close(rc)
    return out


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_native_prompt_steps_match_the_parts(name, tmp_path):
    folder = make_folder(name, str(tmp_path))
    cfg, w = plain_model.read_folder(folder)
    rng = random.Random(11)
    seqs = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (150, 97, 40)]
    cuts = [70, 33, 20, 200]
    native, parts = runner_for(folder, True), runner_for(folder, False)
    assert native.model.native_prompt is not None
    a = run_portions(native, seqs, cuts)
    b = run_portions(parts, seqs, cuts)
    assert native.model.native_prompt.steps >= 3          # the steps of more than 16 tokens went through it
    want = [plain_model.forward(cfg, w, s).numpy() for s in seqs]
    scale = max(float(np.abs(x).max()) for x in want)
    assert a.keys() == b.keys() and len(a) == 7
    for (i, pos), row in a.items():
        assert np.isfinite(row).all()
        assert np.abs(row - b[(i, pos)]).max() <= 2e-2 * scale        # the bias is rounded once more
        assert np.abs(row - want[i][pos]).max() <= 3e-2 * scale
    native.cache.check()


def test_native_prompt_declines_float32(tmp_path):
    """The native loop is for bfloat16; the float32 path keeps the parts' own launches."""
    from qwen_decoder_b200.engine import ModelRunner
    r32 = ModelRunner.from_folder(make_folder("A", str(tmp_path)), dtype="float32", device="cuda:0",
                                  num_pages=16, page_size=16, max_requests=2)
    assert r32.model.native_prompt is None
