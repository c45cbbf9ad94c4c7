"""Each part alone -- norm, position encoding, feed-forward, mixer, block -- built through the registry,
bound to random tensors and run on a step's tokens, against the plain implementation; at sizes other than
the tiny configurations', in float32 and in bfloat16, for a few tokens (the decode kernels) and for many
(the prompt kernels)."""
import math

import pytest
import torch

import plain_model
from qwen_decoder_b200.cache import CacheLayout, CacheManager
from qwen_decoder_b200.config.registry import create_part
from qwen_decoder_b200.engine.batch import StepEntry, build_context
from qwen_decoder_b200.parts.base import PagedCacheView, ResidualStream
from qwen_decoder_b200.weights.loader import TensorSource

# every device buffer these tests and the code under test allocate lies between guard regions (conftest.py)
pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("guard_regions")]
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 1e-5, torch.bfloat16: 3e-2}


def bind(part, dtype, seed, scale=0.08):
    """Random tensors for every spec of ``part`` (norm scales around one), bound; returns them in float64."""
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for spec in part.tensor_specs():
        t = torch.randn(spec.shape, generator=g) * scale
        if spec.init == "around_one":
            t = 1.0 + t
        tensors[spec.name] = t.to(torch.bfloat16)          # what a checkpoint would hold
    part.bind(TensorSource.from_dict(tensors), dtype, DEV)
    return {n: t.double() for n, t in tensors.items()}


def close(got, want, dtype):
    got, want = got.double().cpu(), want.double()
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= TOL[dtype] * max(1.0, float(want.abs().max()))


def total(delta):
    """A branch output is [T, D], or float32 partial sums [parts, T, D] that the next norm adds up."""
    return delta.sum(0) if delta.dim() == 3 else delta


class FakeContext:
    """What a feed-forward may look at: nothing but the token count."""
    def __init__(self, n):
        self.num_tokens = n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [3, 150])
def test_rmsnorm_part_adds_the_pending_branch(dtype, T):
    D, eps = 200, 3e-5
    norm = create_part("norm", "rmsnorm", size=D, eps=eps, prefix="n.")
    w = bind(norm, dtype, 1)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, D, generator=g)
    for delta in (None, torch.randn(T, D, generator=g).to(dtype), torch.randn(3, T, D, generator=g)):
        stream = ResidualStream(x.clone().to(DEV))
        if delta is not None:
            stream.push(delta.to(DEV))
        out = norm.forward(stream, dtype)
        summed = x.double() + (total(delta).double() if delta is not None else 0.0)
        close(stream.x, summed, torch.float32)                         # the residual sum stays float32
        close(out, plain_model.rmsnorm(summed, w["n.weight"], eps), dtype)
        assert stream.delta is None and out.dtype == dtype


def test_rotary_part_tables():
    d, base = 96, 12345.0
    rot = create_part("position", "rotary", head_dim=d, rotary_dim=d, base=base, pairing="adjacent")
    rot.prepare(500, DEV)
    p = torch.arange(d // 2, dtype=torch.float64)
    angle = torch.arange(500, dtype=torch.float64)[:, None] / base ** (2.0 * p / d)[None, :]
    assert rot.cos.shape == (500, d // 2) and rot.cos.dtype == torch.float32
    assert (rot.cos.double().cpu() - angle.cos()).abs().max() < 1e-6
    assert (rot.sin.double().cpu() - angle.sin()).abs().max() < 1e-6
    with pytest.raises(ValueError):
        create_part("position", "rotary", head_dim=d, rotary_dim=d + 2, base=base)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [1, 6, 40, 300])
def test_swiglu_part(dtype, T):
    D, F = 192, 520
    ff = create_part("feed_forward", "swiglu", hidden_size=D, intermediate_size=F, prefix="m.")
    w = bind(ff, dtype, 3)
    x = torch.randn(T, D, generator=torch.Generator().manual_seed(4)).to(dtype)
    got = total(ff.forward(x.to(DEV), FakeContext(T)))
    want = plain_model.swiglu_ffn(x.double(), w["m.gate_proj.weight"], w["m.up_proj.weight"], w["m.down_proj.weight"])
    close(got, want, dtype)


@pytest.mark.parametrize("T,D,F", [(1, 3080, 264), (8, 2056, 520), (8, 1032, 1100), (9, 1032, 520), (13, 3080, 260),
                                   (16, 192, 2200), (17, 264, 520)])
def test_swiglu_part_at_every_few_token_form(T, D, F):
    """bfloat16 at the token counts and widths where the feed-forward changes its kernels: one launch (up to 8
    tokens, hidden size up to 2,048), gate/up as partial sums with a SwiGLU kernel of its own (up to 8 tokens and
    a wider hidden size; 9 to 16 tokens), the library product from 17 tokens on.  Tokens 8.. differ in scale from
    tokens 0..7."""
    dtype = torch.bfloat16
    ff = create_part("feed_forward", "swiglu", hidden_size=D, intermediate_size=F, prefix="m.")
    w = bind(ff, dtype, 5, scale=0.04)
    x = torch.randn(T, D, generator=torch.Generator().manual_seed(6))
    x[8:] *= 2.0
    x = x.to(dtype)
    got = total(ff.forward(x.to(DEV), FakeContext(T)))
    want = plain_model.swiglu_ffn(x.double(), w["m.gate_proj.weight"], w["m.up_proj.weight"], w["m.down_proj.weight"])
    close(got, want, dtype)


def attention_setup(dtype, H, G, d, D, window, page_size=16):
    rot = create_part("position", "rotary", head_dim=d, rotary_dim=d, base=30000.0, pairing="adjacent")
    rot.prepare(600, DEV)
    mixer = create_part("mixer", "gq_attention", hidden_size=D, num_heads=H, num_kv_heads=G, head_dim=d,
                        qkv_bias=True, out_bias=False, position=rot, window=window, prefix="a.")
    w = bind(mixer, dtype, 5)
    cache = CacheManager(CacheLayout.from_needs([mixer.cache_need()], [None]), 64, page_size, 4, dtype=dtype, device=DEV)
    return mixer, w, cache


def plain_attention(x, w, H, G, d, window):
    cfg = {"num_attention_heads": H, "num_key_value_heads": G, "head_dim": d, "hidden_size": x.shape[1],
           "rope_theta": 30000.0, "rope_pairing": "adjacent"}
    ww = {k.replace("a.", "L.self_attn."): v for k, v in w.items()}
    return plain_model.attention_block(x, ww, "L.", cfg, torch.arange(x.shape[0]), window)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(6, 2, 64, 136, None), (5, 5, 48, 104, 37), (8, 1, 128, 160, None)])
def test_attention_part_with_its_cache(dtype, shape):
    """The mixer alone: a prompt portion, a second portion that reads the first from the cache, then single
    tokens -- the same part object takes the prompt kernels and the decode kernels."""
    H, G, d, D, window = shape
    mixer, w, cache = attention_setup(dtype, H, G, d, D, window)
    n = 150
    x = torch.randn(n, D, generator=torch.Generator().manual_seed(6)).to(dtype)
    want = plain_attention(x.double(), w, H, G, d, window)
    rc = cache.open("r")
    got = []
    start = 0
    for count in (70, 61, 1, 1, 2, 15):            # two portions, single tokens, two more portions
        cache.ensure(rc, start + count)
        ctx = build_context([StepEntry(rc, [0] * count, [])], cache, DEV, 10, 600)
        view = PagedCacheView(kv=cache.layer_kv(0), group=ctx.groups[0], write=True)
        got.append(total(mixer.forward(x[start:start + count].to(DEV), ctx, view)).float().cpu())
        cache.commit(rc, count)
        start += count
    close(torch.cat(got), want, dtype)
    cache.close(rc)
    cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block(dtype):
    """The block's arrangement: x += mixer(norm(x)); x += feed_forward(norm(x)), the second branch left
    pending on the stream."""
    H, G, d, D, F, eps = 4, 2, 32, 88, 240, 1e-5
    mixer, wa, cache = attention_setup(dtype, H, G, d, D, None)
    ff = create_part("feed_forward", "swiglu", hidden_size=D, intermediate_size=F, prefix="m.")
    n1 = create_part("norm", "rmsnorm", size=D, eps=eps, prefix="n1.")
    n2 = create_part("norm", "rmsnorm", size=D, eps=eps, prefix="n2.")
    wf, w1, w2 = bind(ff, dtype, 7), bind(n1, dtype, 8), bind(n2, dtype, 9)
    block = create_part("block", "pre_norm", mixer=mixer, feed_forward=ff, norms={"input": n1, "post_mixer": n2})
    block.dtype = dtype
    n = 45
    x = torch.randn(n, D, generator=torch.Generator().manual_seed(10))
    rc = cache.open("r")
    cache.ensure(rc, n)
    ctx = build_context([StepEntry(rc, [0] * n, [])], cache, DEV, 10, 600)
    stream = ResidualStream(x.clone().to(DEV))
    block.forward(stream, ctx, PagedCacheView(kv=cache.layer_kv(0), group=ctx.groups[0], write=True))
    assert stream.delta is not None
    stream.flush()
    xd = x.double()
    xd = xd + plain_attention(plain_model.rmsnorm(xd, w1["n1.weight"], eps), wa, H, G, d, None)
    h = plain_model.rmsnorm(xd, w2["n2.weight"], eps)
    xd = xd + plain_model.swiglu_ffn(h, wf["m.gate_proj.weight"], wf["m.up_proj.weight"], wf["m.down_proj.weight"])
    close(stream.x, xd, dtype)
