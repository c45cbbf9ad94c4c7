"""The plain implementation itself: against logits made by the reference project's own CPU forward
(tests/golden/), and properties of its parts."""
import math
import os
import sys

import numpy as np
import pytest
import torch

import plain_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)
import golden_model  # noqa: E402


def test_plain_forward_equals_the_reference_cpu_decoder():
    """reference_cpu_logits.npy was written by make_golden.py from the reference's cpu_decoder.cpp
    (float32, token by token, its own cache); the plain implementation (float64, whole sequence, no
    cache) must give the same logits up to float32 rounding."""
    want = np.load(os.path.join(GOLDEN, "reference_cpu_logits.npy"))
    w = {k: torch.from_numpy(v) for k, v in golden_model.weights().items()}
    got = plain_model.forward(golden_model.CONFIG, w, golden_model.TOKENS).numpy()
    assert got.shape == want.shape
    err = np.abs(got - want).max()
    assert err <= 2e-6 * np.abs(want).max(), err
    assert (got.argmax(-1) == want.argmax(-1)).all()


def test_half_split_pairs_another_eps_and_one_kv_head_on_the_reference_cpu_decoder():
    """reference_cpu_logits_b.npy: the reference's CPU forward on a model that is equivalent, by a reordering
    of the rows of Wq and Wk and a scaling of the matrices that write to the residual sum, to one with
    half-split rotary pairs and eps 1e-5 (golden_model.py says why).  The plain implementation computes
    that model directly, with ``rope_pairing`` "half" and its own eps."""
    want = np.load(os.path.join(GOLDEN, "reference_cpu_logits_b.npy"))
    cfg = golden_model.CONFIG_B
    assert cfg["rope_pairing"] == "half" and cfg["rms_norm_eps"] == 1e-5 and cfg["num_key_value_heads"] == 1
    w = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in golden_model.weights_b().items()}
    got = plain_model.forward(cfg, w, golden_model.TOKENS_B).numpy()
    assert got.shape == want.shape
    err = np.abs(got - want).max()
    assert err <= 2e-6 * np.abs(want).max(), err
    # and it does pin them: the other pairing or the reference's eps on the same tensors is another function
    for other in (dict(cfg, rope_pairing="adjacent"), dict(cfg, rms_norm_eps=1e-6)):
        assert np.abs(plain_model.forward(other, w, golden_model.TOKENS_B).numpy() - want).max() > 1e-4


def test_half_pairing_is_a_different_function():
    w = {k: torch.from_numpy(v) for k, v in golden_model.weights().items()}
    want = np.load(os.path.join(GOLDEN, "reference_cpu_logits.npy"))
    got = plain_model.forward(dict(golden_model.CONFIG, rope_pairing="half"), w, golden_model.TOKENS).numpy()
    assert np.abs(got - want).max() > 1e-4          # so the test above does pin the pairing


def test_rmsnorm_and_silu():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    out = plain_model.rmsnorm(x, torch.tensor([1.0, 2.0], dtype=torch.float64), 0.0)
    assert torch.allclose(out, torch.tensor([[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]], dtype=torch.float64))
    assert abs(float(plain_model.silu(torch.tensor(1.0, dtype=torch.float64))) - 1 / (1 + math.exp(-1))) < 1e-15


def test_rope_rotates_pairs_and_keeps_position_zero():
    x = torch.arange(16, dtype=torch.float64).reshape(1, 16) + 1
    assert torch.equal(plain_model.rope(x, torch.tensor([0]), 2, 8, 10000.0), x)
    y = plain_model.rope(x, torch.tensor([3]), 2, 8, 10000.0, "adjacent")
    a = 3.0          # pair 0 of each head turns by pos * base^0
    assert abs(float(y[0, 0]) - (1 * math.cos(a) - 2 * math.sin(a))) < 1e-12
    assert abs(float(y[0, 9]) - (9 * math.sin(a) + 10 * math.cos(a))) < 1e-12
    z = plain_model.rope(x, torch.tensor([3]), 2, 8, 10000.0, "half")
    assert abs(float(z[0, 0]) - (1 * math.cos(a) - 5 * math.sin(a))) < 1e-12
    # norms of pairs are kept
    assert abs(float((y ** 2).sum() - (x ** 2).sum())) < 1e-9


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(0)
    T, H, G, d = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n * d, generator=g, dtype=torch.float64) for n in (H, G, G))
    out = plain_model.attention(q, k, v, H, G, d)
    assert torch.allclose(out[0].reshape(H, d), v[0].reshape(G, d).repeat_interleave(2, 0))   # one key
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0, 0
    assert torch.allclose(plain_model.attention(q, k2, v2, H, G, d)[:5], out[:5])             # causal
    w = plain_model.attention(q, k, v, H, G, d, window=3)
    assert torch.allclose(w[:3], out[:3]) and not torch.allclose(w[5], out[5])
    k3, v3 = k.clone(), v.clone()
    k3[:6], v3[:6] = 7, 7
    assert torch.allclose(plain_model.attention(q, k3, v3, H, G, d, window=3)[8], w[8])       # keys 6..8 only


def test_sampler_follows_the_reference_rules():
    l = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert plain_model.argmax(l) == 1                                     # first maximum
    assert plain_model.sample_topk(l, 0, 0.0, 0.9)[0] == 1
    p = torch.softmax(l.double() / 0.5, 0)
    assert plain_model.sample_topk(l, 0, 0.5, float(p[0]) * 0.5)[0] == 0
    assert plain_model.sample_topk(l, 0, 0.5, float(p[0] + p[1] * 0.5))[0] == 1
    assert plain_model.sample_topk(l, 2, 0.5, 0.75)[0] == 2               # top-2 keeps the two 2.0s
    assert plain_model.sample_topk(l, 1, 0.5, 0.75)[0] == 2               # ties at the threshold are kept
    assert plain_model.sample_topk(l, 3, 1.0, 0.999999)[0] == 2
