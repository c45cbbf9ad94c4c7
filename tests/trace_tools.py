"""Building replay traces for tests and checking replayed logits against expectations."""
import io
import json
import os
import random
from typing import Dict, List, Sequence, Tuple

import numpy as np


class Trace:
    """Steps as trace_run reads them, plus for every wanted row which (request, position) it is."""

    def __init__(self):
        self.steps: List[dict] = []
        self.expect: Dict[int, List[Tuple[int, int]]] = {}

    def add(self, entries, end=()):
        """entries: list of (request index, first position, tokens, want places)."""
        s = len(self.steps)
        self.steps.append({
            "step": s,
            "entries": [{"id": f"r{r}", "tokens": list(map(int, toks)), "want": list(map(int, want))}
                        for r, _, toks, want in entries],
            "end": [f"r{r}" for r in end]})
        rows = [(r, p0 + w) for r, p0, _, want in entries for w in want]
        if rows:
            self.expect[s] = rows
        return s

    def lines(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def _wanted(keep, r, p0, n):
    """Places 0..n-1 of a portion that starts at position p0 of request r; ``keep(r, position)`` thins them
    (a model with a large vocabulary wants logits at chosen positions, not at all of them)."""
    return range(n) if keep is None else [i for i in range(n) if keep(r, p0 + i)]


def whole(seqs: Sequence[Sequence[int]], keep=None) -> Trace:
    """Each request alone, whole, logits everywhere."""
    t = Trace()
    for r, seq in enumerate(seqs):
        t.add([(r, 0, seq, _wanted(keep, r, 0, len(seq)))], end=[r])
    return t


def decode_tail(seqs, tail=32, keep=None) -> Trace:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    t = Trace()
    for r, seq in enumerate(seqs):
        n0 = max(1, len(seq) - tail)
        t.add([(r, 0, seq[:n0], _wanted(keep, r, 0, n0))])
        for p in range(n0, len(seq)):
            t.add([(r, p, seq[p:p + 1], [0])], end=[r] if p == len(seq) - 1 else [])
        if n0 == len(seq):
            t.steps[-1]["end"] = [f"r{r}"]
    return t


def portions(seqs, sizes=(7, 2, 24, 3, 2, 16, 5, 2, 31, 2), keep=None) -> Trace:
    """Each request in portions of changing size, down to two tokens."""
    t = Trace()
    for r, seq in enumerate(seqs):
        p, i = 0, r
        while p < len(seq):
            n = min(sizes[i % len(sizes)], len(seq) - p)
            i += 1
            last = p + n == len(seq)
            t.add([(r, p, seq[p:p + n], _wanted(keep, r, p, n))], end=[r] if last else [])
            p += n
    return t


def mixed(seqs, max_tokens: int, seed: int, max_live=4, prompt_frac=0.6, keep=None,
          portion_sizes=(2, 3, 5, 8, 13, 24)) -> Trace:
    """Up to ``max_live`` live requests; some get portions of their prompt (2..24 tokens), others
    single tokens, some sit a step out; a request starts only when the pool (``max_tokens``, each
    request's length rounded up to 64) has room, so pages of finished requests are used again."""
    rng = random.Random(seed)
    t = Trace()
    pending = list(range(len(seqs)))
    live: Dict[int, int] = {}          # request -> tokens fed so far
    held = lambda r: (len(seqs[r]) + 63) // 64 * 64
    while pending or live:
        while pending and len(live) < max_live and sum(held(r) for r in live) + held(pending[0]) <= max_tokens:
            live[pending.pop(0)] = 0
        assert live, "max_tokens too small for the next request"
        entries, end = [], []
        for r in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            p = live[r]
            prompt_len = int(len(seqs[r]) * prompt_frac)
            if p < prompt_len:
                n = min(rng.choice(list(portion_sizes)), len(seqs[r]) - p)
            else:
                n = 1
            entries.append((r, p, seqs[r][p:p + n], _wanted(keep, r, p, n) if n > 1 else [0]))
            live[r] = p + n
            if live[r] == len(seqs[r]):
                end.append(r)
                del live[r]
        if entries:
            t.add(entries, end)
    return t


def run_inprocess(runner, trace: Trace, out_dir: str) -> Dict[int, np.ndarray]:
    """Replay through the engine's own replay loop; returns step -> [rows, vocab]."""
    from qwen_decoder_b200.engine.trace import replay
    done = io.StringIO()
    replay(runner, io.StringIO(trace.lines()), out_dir, done)
    assert done.getvalue().splitlines() == [f"done {s['step']}" for s in trace.steps]
    return read_outputs(trace, out_dir, runner.model.vocab_size)


def read_outputs(trace: Trace, out_dir: str, vocab: int) -> Dict[int, np.ndarray]:
    out = {}
    for s, rows in trace.expect.items():
        a = np.fromfile(os.path.join(out_dir, f"{s}.f32"), dtype="<f4")
        assert a.size == len(rows) * vocab, (s, a.size, len(rows), vocab)
        out[s] = a.reshape(len(rows), vocab)
    return out


def compare(trace: Trace, got: Dict[int, np.ndarray], want_logits, rel_tol: float):
    """Every replayed row against the plain implementation's row; the first wrong place is named.
    ``want_logits[r]`` is indexed by position: an array [positions, vocab] or a dict position -> row."""
    def largest(w):
        return max(float(np.abs(v).max()) for v in w.values()) if isinstance(w, dict) else float(np.abs(w).max())
    scale = max(largest(w) for w in want_logits)
    worst = 0.0
    for s in sorted(trace.expect):
        for i, (r, p) in enumerate(trace.expect[s]):
            err = float(np.abs(got[s][i].astype(np.float64) - want_logits[r][p]).max())
            worst = max(worst, err)
            assert err <= rel_tol * scale, (
                f"step {s} row {i}: request {r} position {p}: max |diff| {err:.3e} > "
                f"{rel_tol:.1e} * {scale:.3e}")
    return worst / scale
