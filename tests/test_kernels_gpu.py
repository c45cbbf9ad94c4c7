"""Each kernel alone against a plain float64 torch reference, at sizes the engine's tiny
models do not use (odd widths, other head sizes, other page sizes)."""
import math

import numpy as np
import pytest
import torch

import plain_model

# every device buffer these tests and the code under test allocate lies between guard regions (conftest.py)
pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("guard_regions")]
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dt):
    return 2e-6 if dt == torch.float32 else 1e-2


# bfloat16 products summed in float32 by the tensor cores: the sum of K terms is not an IEEE sequential
# sum; its error grows like sqrt(K) * 2^-24 (2.7e-6 at K = 2048), bounded here at 1e-5 of the largest result
TENSOR_F32 = "tensor-core float32 accumulation"


def close(got, want, dt, scale=None):
    want = want.to(torch.float64)
    s = float(want.abs().max()) if scale is None else scale
    err = float((got.to(torch.float64).cpu() - want.cpu()).abs().max())
    t = 1e-5 if dt == TENSOR_F32 else tol(dt)
    assert err <= t * max(s, 1e-30), f"max |diff| {err:.3e} vs scale {s:.3e}"


@pytest.mark.parametrize("dt", DTYPES)
def test_embedding(dt):
    from qwen_decoder_b200 import kernels
    g = torch.Generator().manual_seed(0)
    table = torch.randn(301, 72, generator=g).to(dt)
    toks = torch.randint(0, 301, (37,), generator=g, dtype=torch.int32)
    x = torch.empty(37, 72, dtype=torch.float32, device=DEV)
    kernels.embedding(x, table.to(DEV), toks.to(DEV))
    assert torch.equal(x.cpu(), table.float()[toks.long()])


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("D", [72, 1000, 4096])
def test_add_rmsnorm(dt, D):
    from qwen_decoder_b200 import kernels
    g = torch.Generator().manual_seed(1)
    x = torch.randn(19, D, generator=g)
    delta = torch.randn(19, D, generator=g).to(dt)
    w = 1 + 0.1 * torch.randn(D, generator=g)
    eps = 3e-5
    xs = x.to(DEV).clone()
    out = torch.empty(19, D, dtype=dt, device=DEV)
    kernels.add_rmsnorm(xs, delta.to(DEV), w.to(DEV), out, eps)
    v = x.double() + delta.double()
    close(xs, v, torch.float32)
    close(out, plain_model.rmsnorm(v, w.double(), eps), dt)
    # gathered rows, no write-back, no delta
    rows = torch.tensor([18, 0, 7], dtype=torch.int32)
    xs2 = x.to(DEV).clone()
    out2 = torch.empty(3, D, dtype=dt, device=DEV)
    kernels.add_rmsnorm(xs2, None, w.to(DEV), out2, eps, rows=rows.to(DEV), write_back=False)
    assert torch.equal(xs2.cpu(), x)
    close(out2, plain_model.rmsnorm(x.double()[rows.long()], w.double(), eps), dt)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("shape", [(1, 40, 24), (7, 130, 99), (70, 65, 257), (129, 200, 64)])
def test_gemm_generic(dt, shape):
    from qwen_decoder_b200 import kernels
    T, N, K = shape
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, K, generator=g).to(dt)
    w = (0.05 * torch.randn(N, K, generator=g)).to(dt)
    b = torch.randn(N, generator=g)
    for bias in (None, b):
        for odt in ([dt] if dt == torch.float32 else [dt, torch.float32]):
            out = torch.empty(T, N, dtype=odt, device=DEV)
            kernels.gemm_generic(x.to(DEV), w.to(DEV), bias.to(DEV) if bias is not None else None, out)
            want = plain_model.linear(x.double(), w.double(), bias.double() if bias is not None else None)
            close(out, want, odt)


def _paged_setup(dt, T_per_req, G, d, page_size, seed):
    """Random pages for requests of the given lengths; returns k, v per request and the device cache."""
    g = torch.Generator().manual_seed(seed)
    n_pages_needed = sum((n + page_size - 1) // page_size for n in T_per_req)
    num_pages = n_pages_needed + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    kv = torch.zeros(num_pages, 2, G, page_size, d, dtype=dt)
    tables, ks, vs = [], [], []
    for n in T_per_req:
        k = torch.randn(n, G, d, generator=g).to(dt)
        v = torch.randn(n, G, d, generator=g).to(dt)
        pages = [perm.pop() for _ in range((n + page_size - 1) // page_size)]
        for t in range(n):
            kv[pages[t // page_size], 0, :, t % page_size, :] = k[t]
            kv[pages[t // page_size], 1, :, t % page_size, :] = v[t]
        tables.append(pages)
        ks.append(k)
        vs.append(v)
    mb = max(len(p) for p in tables)
    bt = torch.full((len(tables), mb), -1, dtype=torch.int32)
    for i, p in enumerate(tables):
        bt[i, :len(p)] = torch.tensor(p, dtype=torch.int32)
    return kv, bt, ks, vs


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg", [(4, 2, 16, 16, None), (6, 2, 48, 8, None), (8, 1, 128, 32, None),
                                 (3, 3, 80, 16, 37), (2, 1, 256, 16, None)])
def test_paged_attention_generic(dt, cfg):
    from qwen_decoder_b200 import kernels
    H, G, d, page_size, window = cfg
    lens = [70, 1, 33]
    kv, bt, ks, vs = _paged_setup(dt, lens, G, d, page_size, seed=3)
    g = torch.Generator().manual_seed(4)
    # queries: the last 5 positions of request 0 (a portion), position 0 of request 1, all of request 2
    items = [(0, p) for p in range(65, 70)] + [(1, 0)] + [(2, p) for p in range(33)]
    q = torch.randn(len(items), H * d, generator=g).to(dt)
    # one query and one far key scaled so that a single score stands out among many
    q[2] *= 4.0
    out = torch.empty(len(items), H * d, dtype=dt, device=DEV)
    tr = torch.tensor([r for r, _ in items], dtype=torch.int32)
    pos = torch.tensor([p for _, p in items], dtype=torch.int32)
    kernels.paged_attention_generic(q.to(DEV), H * d, out, kv.to(DEV), bt.to(DEV), tr.to(DEV), pos.to(DEV),
                                    len(items), H, G, d, page_size, 1.0 / math.sqrt(d), window or 0)
    for i, (r, p) in enumerate(items):
        n = p + 1
        qq = torch.zeros(n, H * d, dtype=torch.float64)
        qq[p] = q[i].double()
        want = plain_model.attention(qq, ks[r][:n].double().reshape(n, G * d), vs[r][:n].double().reshape(n, G * d),
                                     H, G, d, window)[p]
        close(out[i], want, dt, scale=float(vs[r][:n].abs().max()))


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("pairing", ["adjacent", "half"])
def test_rope_kv_write(dt, pairing):
    from qwen_decoder_b200 import kernels
    from qwen_decoder_b200.parts.rotary import Rotary
    H, G, d, page_size, T = 6, 2, 48, 8, 21
    base = 50000.0
    rot = Rotary(d, d, base, pairing)
    rot.prepare(300, torch.device(DEV))
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(T, (H + 2 * G) * d, generator=g).to(dt)
    positions = torch.randint(0, 300, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(5 * page_size, generator=g)[:T].to(torch.int32)
    kv = torch.zeros(5, 2, G, page_size, d, dtype=dt, device=DEV)
    dq = qkv.to(DEV).clone()
    kernels.rope_kv_write(dq, H, G, d, d, rot.pairing_code, rot.cos, rot.sin, positions.to(DEV), kv,
                          slots.to(DEV), page_size, True)
    x = qkv.double()
    wq = plain_model.rope(x[:, :H * d], positions, H, d, base, pairing)
    wk = plain_model.rope(x[:, H * d:(H + G) * d], positions, G, d, base, pairing)
    wv = x[:, (H + G) * d:]
    close(dq[:, :H * d], wq, dt)
    kvc = kv.cpu()
    for t in range(T):
        page, off = int(slots[t]) // page_size, int(slots[t]) % page_size
        close(kvc[page, 0, :, off, :].reshape(-1), wk[t], dt)
        close(kvc[page, 1, :, off, :].reshape(-1), wv[t], dt)


@pytest.mark.parametrize("pairing", ["adjacent", "half"])
@pytest.mark.parametrize("sizes", [(6, 2, 48, 48), (4, 1, 128, 128), (3, 3, 64, 32), (2, 1, 40, 40)])
def test_rope_kv_write_with_bias(pairing, sizes):
    """The vectorized kernel with the projection's bias, both pairings, partly rotated heads; sizes it does
    not take are refused, not computed wrongly."""
    from qwen_decoder_b200 import kernels
    from qwen_decoder_b200.parts.rotary import Rotary
    H, G, d, rd = sizes
    page_size, T, base = 16, 37, 20000.0
    dt = torch.bfloat16
    rot = Rotary(d, rd, base, pairing)
    rot.prepare(400, torch.device(DEV))
    g = torch.Generator().manual_seed(15)
    qkv = torch.randn(T, (H + 2 * G) * d, generator=g).to(dt)
    bias = torch.randn((H + 2 * G) * d, generator=g)
    positions = torch.randint(0, 400, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(4 * page_size, generator=g)[:T].to(torch.int32)
    kv = torch.zeros(4, 2, G, page_size, d, dtype=dt, device=DEV)
    dq = qkv.to(DEV).clone()
    call = lambda: kernels.rope_kv_write_biased(dq, bias.to(DEV), H, G, d, rd, rot.pairing_code, rot.cos, rot.sin,
                                                positions.to(DEV), kv, slots.to(DEV), page_size, True)
    if rd % (8 if pairing == "adjacent" else 16):
        with pytest.raises(kernels.KernelError):
            call()
        return
    call()
    x = (qkv.float() + bias).to(dt).double()           # the sum is rounded to bfloat16 before the rotation

    def rotate(part, heads):
        part = part.reshape(T, heads, d)
        turned = plain_model.rope(part[:, :, :rd].reshape(T, heads * rd), positions, heads, rd, base, pairing)
        return torch.cat([turned.reshape(T, heads, rd), part[:, :, rd:]], dim=2).reshape(T, heads * d)

    wq, wk = rotate(x[:, :H * d], H), rotate(x[:, H * d:(H + G) * d], G)
    wv = x[:, (H + G) * d:]
    close(dq[:, :H * d], wq, dt)
    kvc = kv.cpu()
    for t in range(T):
        page, off = int(slots[t]) // page_size, int(slots[t]) % page_size
        close(kvc[page, 0, :, off, :].reshape(-1), wk[t], dt)
        close(kvc[page, 1, :, off, :].reshape(-1), wv[t], dt)


@pytest.mark.parametrize("dt", DTYPES)
def test_swiglu(dt):
    from qwen_decoder_b200 import kernels
    g = torch.Generator().manual_seed(6)
    gu = (3 * torch.randn(13, 2 * 177, generator=g)).to(dt)
    out = torch.empty(13, 177, dtype=dt, device=DEV)
    kernels.swiglu(gu.to(DEV), out)
    x = gu.double()
    close(out, plain_model.silu(x[:, :177]) * x[:, 177:], dt)


def test_sampling():
    from qwen_decoder_b200 import kernels
    g = torch.Generator().manual_seed(7)
    V = 1531
    R = 64
    logits = 2.0 * torch.randn(R, V, generator=g)
    logits[3, 100] = logits[3, 900] = logits[3].max() + 1.0      # a tie: the lower index wins
    temps = torch.tensor([0.0, 0.7, 1.0, 0.0] * 16)
    ks = torch.tensor([0, 0, 30, 5, 1, 2000, 7, 0] * 8, dtype=torch.int32)
    draws = torch.rand(R, generator=g)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    kernels.sample(logits.to(DEV), temps.to(DEV), ks.to(DEV), draws.to(DEV), out)
    out = out.cpu()
    checked = 0
    for r in range(R):
        tok, margin = plain_model.sample_topk(logits[r], int(ks[r]), float(temps[r]), float(draws[r]))
        if margin < 1e-5:
            continue      # float32 rounding of the running sum could decide this draw either way
        assert int(out[r]) == tok, (r, int(out[r]), tok)
        checked += 1
    assert checked > R // 2 and int(out[3]) == 100


def _plain_attention_row(q_row, k, v, H, G, d, p, window):
    n = p + 1
    qq = torch.zeros(n, H * d, dtype=torch.float64)
    qq[p] = q_row.double()
    return plain_model.attention(qq, k[:n].double().reshape(n, G * d), v[:n].double().reshape(n, G * d),
                                 H, G, d, window)[p]


@pytest.mark.parametrize("cfg", [(16, 2, 128, 16, None, 1), (16, 2, 128, 16, None, 7), (4, 2, 16, 16, None, 3),
                                 (6, 2, 48, 32, None, 2), (14, 2, 64, 64, 300, 5), (5, 5, 96, 16, None, 4),
                                 (32, 2, 32, 16, 50, 2)])
def test_decode_attention_tensor_cores(cfg):
    """One query token per request; contexts that end inside a page, at a page's edge, of one key;
    a window; keys split over several CTAs; one far key made to stand out."""
    _decode_attention_case(cfg)


@pytest.mark.parametrize("cfg", [(16, 2, 128, 16, None, 1), (16, 2, 128, 16, None, 7), (14, 2, 64, 64, 300, 5),
                                 (8, 8, 64, 32, None, 3), (32, 2, 128, 16, 50, 2)])
def test_decode_attention_fed_by_tma(cfg, monkeypatch):
    """The same cases through the kernel that fetches K/V with TMA tensor copies (head sizes 64 and 128)."""
    from qwen_decoder_b200 import kernels
    monkeypatch.setattr(kernels, "_DECODE_TMA", True)
    _decode_attention_case(cfg)
    assert kernels.library("attention_flash").qd_decode_attention_tma_status() == 0


def _decode_attention_case(cfg):
    from qwen_decoder_b200 import kernels
    H, G, d, page_size, window, splits = cfg
    dt = torch.bfloat16
    lens = [1, 16, 17, 255, 256, 700, 1031]
    kv, bt, ks, vs = _paged_setup(dt, lens, G, d, page_size, seed=11)
    g = torch.Generator().manual_seed(12)
    q = torch.randn(len(lens), H * d, generator=g).to(dt)
    # request 5: key 3 (far back) gets a large score for head 0 only
    ks[5][3, 0] = (q[5, :d].float() * 3.0).to(dt)
    page = int(bt[5, 3 // page_size])
    kv[page, 0, 0, 3 % page_size] = ks[5][3, 0]
    out = torch.empty(len(lens), H * d, dtype=dt, device=DEV)
    tr = torch.arange(len(lens), dtype=torch.int32)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    kernels.decode_attention(q.to(DEV), H * d, out, kv.to(DEV), bt.to(DEV), tr.to(DEV), pos.to(DEV), len(lens),
                             H, G, d, page_size, 1.0 / math.sqrt(d), window or 0, splits)
    for i, n in enumerate(lens):
        want = _plain_attention_row(q[i], ks[i], vs[i], H, G, d, n - 1, window)
        close(out[i], want, dt, scale=float(vs[i].abs().max()))
    if window is None and G < H:
        # the far key dominates head 0 of request 5
        assert float((out[5, :d].float().cpu() - vs[5][3, 0].float()).abs().max()) < 0.3


@pytest.mark.parametrize("cfg", [(16, 2, 128, 16, None), (4, 2, 16, 16, None), (6, 2, 48, 8, None),
                                 (4, 1, 32, 32, None), (3, 3, 64, 16, 40), (8, 1, 96, 16, None), (7, 7, 128, 16, 100)])
def test_prefill_attention_tensor_cores(cfg):
    """Portions with and without history, of one token up to hundreds, several requests in a batch."""
    from qwen_decoder_b200 import kernels
    H, G, d, page_size, window = cfg
    dt = torch.bfloat16
    # (cached before, portion): whole prompt, portion after history, single token, two tokens at a page edge
    plan = [(0, 150), (70, 45), (129, 1), (15, 2), (0, 1), (200, 130)]
    lens = [a + b for a, b in plan]
    kv, bt, ks, vs = _paged_setup(dt, lens, G, d, page_size, seed=13)
    g = torch.Generator().manual_seed(14)
    T = sum(b for _, b in plan)
    q = torch.randn(T, H * d, generator=g).to(dt)
    cu = torch.tensor([0] + list(torch.tensor([b for _, b in plan]).cumsum(0)), dtype=torch.int32)
    start = torch.tensor([a for a, _ in plan], dtype=torch.int32)
    out = torch.empty(T, H * d, dtype=dt, device=DEV)
    kernels.prefill_attention(q.to(DEV), H * d, out, kv.to(DEV), bt.to(DEV), cu.to(DEV), start.to(DEV), len(plan), T,
                              H, G, d, page_size, 1.0 / math.sqrt(d), window or 0)
    outc = out.cpu()
    for r, (a, b) in enumerate(plan):
        n = a + b
        qq = torch.zeros(n, H * d, dtype=torch.float64)
        qq[a:] = q[int(cu[r]):int(cu[r + 1])].double()
        want = plain_model.attention(qq, ks[r].double().reshape(n, G * d), vs[r].double().reshape(n, G * d),
                                     H, G, d, window)[a:]
        close(outc[int(cu[r]):int(cu[r + 1])], want, dt, scale=float(vs[r].abs().max()))


@pytest.mark.parametrize("cfg", [(16, 2, 128, 16, None), (8, 8, 128, 32, None), (4, 1, 64, 16, None),
                                 (16, 1, 64, 64, 40), (2, 1, 128, 16, 300),
                                 # groups that do not divide the tile's 128 rows: 7 heads per KV head (Qwen2.5-7B),
                                 # 5 (32B), 6, 3, 12
                                 (28, 4, 128, 16, None), (40, 8, 128, 16, None), (12, 2, 128, 16, 100), (3, 1, 64, 32, None),
                                 (12, 1, 64, 16, None)])
def test_prefill_attention_tcgen05(cfg):
    """The same portions through the tcgen05 kernel (tensor memory accumulators, K/V by TMA from the pages):
    with and without history, one token up to hundreds, several requests, windows, tiles that end inside
    a key tile of 128."""
    from qwen_decoder_b200 import kernels
    H, G, d, page_size, window = cfg
    assert kernels.prefill_tc5_supported(torch.bfloat16, H, G, d, page_size)
    dt = torch.bfloat16
    plan = [(0, 150), (70, 45), (129, 1), (15, 2), (0, 1), (200, 330), (0, 128), (127, 129)]
    lens = [a + b for a, b in plan]
    kv, bt, ks, vs = _paged_setup(dt, lens, G, d, page_size, seed=13)
    g = torch.Generator().manual_seed(14)
    T = sum(b for _, b in plan)
    q = torch.randn(T, H * d, generator=g).to(dt)
    cu = torch.tensor([0] + list(torch.tensor([b for _, b in plan]).cumsum(0)), dtype=torch.int32)
    start = torch.tensor([a for a, _ in plan], dtype=torch.int32)
    out = torch.full((T, H * d), float("nan"), dtype=dt, device=DEV)
    kernels.prefill_attention_tc5(q.to(DEV), H * d, out, kv.to(DEV), bt.to(DEV), cu.to(DEV), start.to(DEV), len(plan),
                                  T, H, G, d, page_size, 1.0 / math.sqrt(d), window or 0)
    assert kernels.prefill_attention_tc5_status() == 0
    outc = out.cpu()
    for r, (a, b) in enumerate(plan):
        n = a + b
        qq = torch.zeros(n, H * d, dtype=torch.float64)
        qq[a:] = q[int(cu[r]):int(cu[r + 1])].double()
        want = plain_model.attention(qq, ks[r].double().reshape(n, G * d), vs[r].double().reshape(n, G * d),
                                     H, G, d, window)[a:]
        close(outc[int(cu[r]):int(cu[r + 1])], want, dt, scale=float(vs[r].abs().max()))


@pytest.mark.parametrize("cfg", [(16, 2, 128, 16), (4, 1, 64, 32), (28, 4, 128, 16)])
def test_prefill_attention_tcgen05_with_a_maximum_that_grows(cfg):
    """The tcgen05 kernel keeps a row's output in tensor memory and rescales it only when the row's maximum has
    grown by more than 2^8 since the reference of its exponentials.  Keys are placed so that rows see both: a
    maximum that creeps up tile by tile (key norms grow along the sequence) and two far keys, in the second
    and in the fourth key tile, whose scores for the last tokens of one head exceed everything before by far
    more than that step; one early key that dominates another head from the first tile on."""
    from qwen_decoder_b200 import kernels
    H, G, d, page_size = cfg
    dt = torch.bfloat16
    plan = [(0, 700), (300, 340)]
    lens = [a + b for a, b in plan]
    kv, bt, ks, vs = _paged_setup(dt, lens, G, d, page_size, seed=31)
    g = torch.Generator().manual_seed(32)
    T = sum(b for _, b in plan)
    q = torch.randn(T, H * d, generator=g).to(dt)
    cu = [0, plan[0][1], T]

    def put(r, key, kv_head, value):              # K of one key of request r, in the list and in its page
        ks[r][key, kv_head] = value.to(dt)
        kv[int(bt[r, key // page_size]), 0, kv_head, key % page_size] = ks[r][key, kv_head]

    for r, (a, b) in enumerate(plan):
        n = a + b
        for key in range(n):                      # norms grow by a factor of three along the sequence
            for kh in range(G):
                put(r, key, kh, ks[r][key, kh].float() * (1.0 + 2.0 * key / n))
        last = q[cu[r + 1] - 1].float()           # the request's last token
        put(r, 140, 0, last[:d] * 1.0)            # head 0: score about sqrt(d) at key 140 ...
        put(r, 400, 0, last[:d] * 2.5)            # ... and 2.5 sqrt(d) at key 400
        put(r, 5, G - 1, last[(H - 1) * d:] * 3.0)     # the last head: its maximum is in the first tile
    out = torch.full((T, H * d), float("nan"), dtype=dt, device=DEV)
    kernels.prefill_attention_tc5(q.to(DEV), H * d, out, kv.to(DEV), bt.to(DEV), torch.tensor(cu, dtype=torch.int32, device=DEV),
                                  torch.tensor([a for a, _ in plan], dtype=torch.int32, device=DEV), len(plan), T, H, G, d,
                                  page_size, 1.0 / math.sqrt(d), 0)
    assert kernels.prefill_attention_tc5_status() == 0
    outc = out.cpu()
    for r, (a, b) in enumerate(plan):
        n = a + b
        qq = torch.zeros(n, H * d, dtype=torch.float64)
        qq[a:] = q[cu[r]:cu[r + 1]].double()
        want = plain_model.attention(qq, ks[r].double().reshape(n, G * d), vs[r].double().reshape(n, G * d), H, G, d, None)[a:]
        close(outc[cu[r]:cu[r + 1]], want, dt, scale=float(vs[r].abs().max()))
        # the far key takes all of head 0 of the last token, the early key all of the last head
        assert float((outc[cu[r + 1] - 1, :d].float() - vs[r][400, 0].float()).abs().max()) < 0.05
        assert float((outc[cu[r + 1] - 1, (H - 1) * d:].float() - vs[r][5, G - 1].float()).abs().max()) < 0.05


@pytest.mark.parametrize("shape", [(1, 48, 64), (7, 130, 72), (8, 2048, 2048), (9, 100, 136), (16, 64, 1000),
                                   (33, 257, 264), (64, 96, 512)])
def test_gemm_skinny(shape):
    """The few-token weight-streaming kernel: every epilogue, sizes that are no multiple of its tiles."""
    from qwen_decoder_b200 import kernels
    T, N, K = shape
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(21)
    x = torch.randn(T, K, generator=g).to(dt)
    w = (0.05 * torch.randn(N, K, generator=g)).to(dt)
    b = torch.randn(N, generator=g)
    want = plain_model.linear(x.double(), w.double())
    for odt in (dt, torch.float32):
        for bias in (None, b):
            out = torch.empty(T, N, dtype=odt, device=DEV)
            kernels.gemm_skinny(x.to(DEV), w.to(DEV), bias.to(DEV) if bias is not None else None, out)
            close(out, want + (bias.double() if bias is not None else 0), odt if odt == dt else TENSOR_F32,
                  scale=float(want.abs().max()) + 1)
    for splits in (1, 3):
        if kernels.few_token_impl(T) == "stream":
            splits = min(splits, (K + 1023) // 1024)      # the streaming kernel splits K in whole stages of 1024
        elif kernels.few_token_impl(T) in ("tc5", ""):
            splits = min(splits, (K + 63) // 64)          # the tcgen05 kernel in whole blocks of 64
        part = kernels.gemm_skinny_partial(x.to(DEV), w.to(DEV), splits)
        assert part.shape == (splits, T, N)
        close(part.sum(0), want, TENSOR_F32, scale=float(want.abs().max()))
    # x as a column slice of a wider buffer (row stride > K)
    wide = torch.zeros(T, K + 64, dtype=dt)
    wide[:, 32:32 + K] = x
    xs = wide.to(DEV)[:, 32:32 + K]
    out = torch.empty(T, N, dtype=torch.float32, device=DEV)
    kernels.gemm_skinny(xs, w.to(DEV), None, out)
    close(out, want, TENSOR_F32, scale=float(want.abs().max()))
    if N % 2 == 0:
        F = N // 2
        h = torch.empty(T, F, dtype=dt, device=DEV)
        kernels.gemm_skinny_swiglu(x.to(DEV), w.to(DEV), h)
        close(h, plain_model.silu(want[:, :F]) * want[:, F:], dt)


@pytest.mark.parametrize("shape", [(9, 100, 136), (12, 2560, 2048), (16, 50, 1000), (16, 2048, 11008), (13, 264, 3080),
                                   (16, 33, 1032)])
def test_gemm_stream_with_sixteen_tokens_resident(shape):
    """9 to 16 tokens through the streaming kernel with the tokens' rows resident: partial sums over shares of one
    stage of K each; a K that is no multiple of a stage, an N that is no multiple of a tile, token rows 8..15 with
    values of their own (a kernel that read rows 0..7 twice would fail), and the feed-forward's SwiGLU from the sums."""
    from qwen_decoder_b200 import kernels
    T, N, K = shape
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(23)
    x = torch.randn(T, K, generator=g)
    x[8:] *= 3.0                                  # the second token tile is not a copy of the first
    x = x.to(dt)
    w = (0.05 * torch.randn(N, K, generator=g)).to(dt)
    want = plain_model.linear(x.double(), w.double())
    shares = kernels.stream_resident_shares(T, K)
    assert shares == (K + 1023) // 1024 and kernels._impl_for(T, K, shares, kernels.EPI_PARTIAL) == "stream"
    assert kernels.skinny_splits(N, K, T) == shares
    wide = torch.zeros(T, K + 64, dtype=dt)       # rows further apart than K
    wide[:, 32:32 + K] = x
    for xin in (x.to(DEV), wide.to(DEV)[:, 32:32 + K]):
        part = kernels.gemm_skinny_partial(xin, w.to(DEV), shares)
        assert kernels.gemm_stream_status() == 0 and part.shape == (shares, T, N)
        close(part.sum(0), want, TENSOR_F32, scale=float(want.abs().max()))
    if N % 8 == 0:
        F = N // 2
        h = torch.full((T, F), float("nan"), dtype=dt, device=DEV)
        kernels.swiglu_partial(part, h)
        close(h, plain_model.silu(want[:, :F]) * want[:, F:], dt)


def test_swiglu_from_partial_sums():
    from qwen_decoder_b200 import kernels
    g = torch.Generator().manual_seed(24)
    for n_parts, T, F in ((1, 3, 8), (2, 16, 1004), (5, 11, 260), (9, 1, 12)):
        part = 2 * torch.randn(n_parts, T, 2 * F, generator=g)
        out = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.swiglu_partial(part.to(DEV), out)
        v = part.double().sum(0)
        close(out, plain_model.silu(v[:, :F]) * v[:, F:], torch.bfloat16)


def test_partial_sums_are_added_by_the_consumers():
    """add_rmsnorm and rope_kv_write_partial take float32 partial sums [parts, T, width]."""
    from qwen_decoder_b200 import kernels
    from qwen_decoder_b200.parts.rotary import Rotary
    g = torch.Generator().manual_seed(22)
    T, D = 5, 200
    x = torch.randn(T, D, generator=g)
    parts = torch.randn(3, T, D, generator=g)
    w = 1 + 0.1 * torch.randn(D, generator=g)
    xs = x.to(DEV).clone()
    out = torch.empty(T, D, dtype=torch.bfloat16, device=DEV)
    kernels.add_rmsnorm(xs, parts.to(DEV), w.to(DEV), out, 1e-6)
    v = x.double() + parts.double().sum(0)
    close(xs, v, torch.float32)
    close(out, plain_model.rmsnorm(v, w.double(), 1e-6), torch.bfloat16)
    xs2 = x.to(DEV).clone()
    kernels.residual_add(xs2, parts.to(DEV))
    close(xs2, v, torch.float32)
    H, G, d, page_size = 6, 2, 48, 16
    W = (H + 2 * G) * d
    rot = Rotary(d, d, 1234.0, "adjacent")
    rot.prepare(100, torch.device(DEV))
    qp = torch.randn(2, T, W, generator=g)
    bias = torch.randn(W, generator=g)
    positions = torch.tensor([0, 5, 99, 31, 32], dtype=torch.int32)
    slots = torch.tensor([3, 17, 40, 41, 0], dtype=torch.int32)
    kv = torch.zeros(3, 2, G, page_size, d, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(T, H * d, dtype=torch.bfloat16, device=DEV)
    kernels.rope_kv_write_partial(qp.to(DEV), bias.to(DEV), q_out, H, G, d, d, 0, rot.cos, rot.sin, positions.to(DEV),
                                  kv, slots.to(DEV), page_size, True)
    full = qp.double().sum(0) + bias.double()
    close(q_out, plain_model.rope(full[:, :H * d], positions, H, d, 1234.0), torch.bfloat16)
    wk = plain_model.rope(full[:, H * d:(H + G) * d], positions, G, d, 1234.0)
    kvc = kv.cpu()
    for t in range(T):
        page, off = int(slots[t]) // page_size, int(slots[t]) % page_size
        close(kvc[page, 0, :, off, :].reshape(-1), wk[t], torch.bfloat16)
        close(kvc[page, 1, :, off, :].reshape(-1), full[t, (H + G) * d:], torch.bfloat16)


@pytest.mark.parametrize("impl", ["stream", "regs", "tc5"])
def test_gemm_skinny_both_implementations(impl, monkeypatch):
    """The persistent bulk-copy streamer, the register-load kernel and the tcgen05 kernel give the same
    products."""
    from qwen_decoder_b200 import kernels
    monkeypatch.setattr(kernels, "skinny_impl", impl)
    for shape in [(1, 48, 64), (8, 2048, 2048), (5, 130, 1096), (16, 22, 2560), (16, 704, 520), (40, 96, 1032)]:
        test_gemm_skinny(shape)
    # many items per persistent CTA, K split in shares: every stage of the ring is reused many times
    g = torch.Generator().manual_seed(23)
    T, N, K = 8, 16 * 700, 3072
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
    want = plain_model.linear(x.double(), w.double())
    part = kernels.gemm_skinny_partial(x.to(DEV), w.to(DEV), 3)
    close(part.sum(0), want, TENSOR_F32, scale=float(want.abs().max()))
    h = torch.empty(T, N // 2, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_skinny_swiglu(x.to(DEV), w.to(DEV), h)
    close(h, plain_model.silu(want[:, :N // 2]) * want[:, N // 2:], torch.bfloat16)
    assert kernels.gemm_stream_status() == 0 and kernels.gemm_tc5_status() == 0


@pytest.mark.parametrize("shape", [(200, 384, 256), (700, 1000, 1096), (129, 130, 72), (2048, 512, 512)])
def test_gemm_tcgen05_many_tokens(shape, monkeypatch):
    """The tcgen05 + TMA kernel with token tiles of 128 and 256: stores with bias, SwiGLU, sizes that are
    no multiple of its tiles (TMA fills what lies outside with zeros)."""
    from qwen_decoder_b200 import kernels
    monkeypatch.setattr(kernels, "skinny_impl", "tc5")
    T, N, K = shape
    g = torch.Generator().manual_seed(24)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    want = plain_model.linear(x.double(), w.double())
    out = torch.empty(T, N, dtype=torch.float32, device=DEV)
    kernels.gemm_skinny(x.to(DEV), w.to(DEV), b.to(DEV), out)
    close(out, want + b.double(), TENSOR_F32, scale=float(want.abs().max()) + 1)
    out16 = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_skinny(x.to(DEV), w.to(DEV), None, out16)
    close(out16, want, torch.bfloat16)
    if N % 2 == 0:
        h = torch.empty(T, N // 2, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_skinny_swiglu(x.to(DEV), w.to(DEV), h)
        close(h, plain_model.silu(want[:, :N // 2]) * want[:, N // 2:], torch.bfloat16)
    assert kernels.gemm_tc5_status() == 0


@pytest.mark.parametrize("cfg", [(16, 2, 128, 16, None, 1, "adjacent"), (16, 2, 128, 16, None, 9, "adjacent"),
                                 (4, 2, 16, 16, None, 3, "half"), (6, 2, 48, 32, None, 2, "half"),
                                 (14, 2, 64, 64, 300, 5, "adjacent"), (5, 5, 96, 16, None, 4, "adjacent"),
                                 (32, 2, 32, 16, 50, 2, "half")])
def test_decode_attention_from_partial_sums(cfg):
    """The kernel that takes q, k, v as float32 partial sums: bias, rotation, cache write and attention in
    one launch, against the plain rotation and attention; the new token's k and v must be in its slot."""
    from qwen_decoder_b200 import kernels
    from qwen_decoder_b200.parts.rotary import Rotary
    H, G, d, page_size, window, splits, pairing = cfg
    dt = torch.bfloat16
    base = 50000.0
    lens = [1, 16, 17, 255, 256, 700, 1031]          # cached length after this step, the new token included
    T, W = len(lens), (H + 2 * G) * d
    rot = Rotary(d, d, base, pairing)
    rot.prepare(1100, torch.device(DEV))
    kv, bt, ks, vs = _paged_setup(dt, lens, G, d, page_size, seed=21)
    g = torch.Generator().manual_seed(22)
    part = torch.randn(3, T, W, generator=g) * 0.6
    bias = torch.randn(W, generator=g) * 0.3
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    slots = torch.tensor([int(bt[i, (n - 1) // page_size]) * page_size + (n - 1) % page_size
                          for i, n in enumerate(lens)], dtype=torch.int32)
    # the slot of the new token holds junk before the step
    for i, n in enumerate(lens):
        kv[int(slots[i]) // page_size, :, :, int(slots[i]) % page_size, :] = 7.0
    qkv = part.double().sum(0) + bias.double()
    wq = plain_model.rope(qkv[:, :H * d], pos, H, d, base, pairing)
    wk = plain_model.rope(qkv[:, H * d:(H + G) * d], pos, G, d, base, pairing).to(dt)
    wv = qkv[:, (H + G) * d:].to(dt)
    dkv = kv.to(DEV)
    out = torch.empty(T, H * d, dtype=dt, device=DEV)
    tr = torch.arange(T, dtype=torch.int32)
    kernels.decode_attention_rope(part.to(DEV), bias.to(DEV), out, dkv, bt.to(DEV), tr.to(DEV), pos.to(DEV),
                                  slots.to(DEV), H, G, d, page_size, 1.0 / math.sqrt(d), window or 0, splits, True,
                                  d, rot.pairing_code, rot.cos, rot.sin)
    kvc = dkv.cpu()
    for i, n in enumerate(lens):
        page, off = int(slots[i]) // page_size, int(slots[i]) % page_size
        close(kvc[page, 0, :, off, :].reshape(-1), wk[i].double(), dt)
        close(kvc[page, 1, :, off, :].reshape(-1), wv[i].double(), dt)
        k_all = torch.cat([ks[i][:n - 1].reshape(n - 1, G, d), wk[i].reshape(1, G, d)])
        v_all = torch.cat([vs[i][:n - 1].reshape(n - 1, G, d), wv[i].reshape(1, G, d)])
        want = _plain_attention_row(wq[i], k_all, v_all, H, G, d, n - 1, window)
        close(out[i], want, dt, scale=float(v_all.abs().max()))
    # reading another layer's cache: nothing is written, the slot's old content is attended
    dkv2 = kv.to(DEV)
    kernels.decode_attention_rope(part.to(DEV), bias.to(DEV), out, dkv2, bt.to(DEV), tr.to(DEV), pos.to(DEV),
                                  slots.to(DEV), H, G, d, page_size, 1.0 / math.sqrt(d), window or 0, splits, False,
                                  d, rot.pairing_code, rot.cos, rot.sin)
    assert torch.equal(dkv2.cpu(), kv)
    # every row, the short ones too: there the chunk with the token's own slot is among the first that a warp
    # asks for, and it may be read only after the kernel before this one has ended
    for i, n in enumerate(lens):
        k_all = torch.cat([ks[i][:n - 1].reshape(n - 1, G, d), torch.full((1, G, d), 7.0, dtype=dt)])
        v_all = torch.cat([vs[i][:n - 1].reshape(n - 1, G, d), torch.full((1, G, d), 7.0, dtype=dt)])
        want = _plain_attention_row(wq[i], k_all, v_all, H, G, d, n - 1, window)
        close(out[i], want, dt, scale=7.0)


@pytest.mark.parametrize("shape", [(8, 2048, 11008), (5, 96, 264), (1, 64, 176), (7, 1024, 2816), (3, 128, 1400)])
def test_feed_forward_in_one_launch(shape):
    """Gate/up with SwiGLU, the wait for the columns of h a CTA's share of the down projection reads, the down
    projection: against the two separate launches and against float64; several times in a row (the
    synchronisation words must be left ready for the next launch)."""
    from qwen_decoder_b200 import kernels
    T, D, F = shape
    g = torch.Generator().manual_seed(31)
    x = (torch.randn(T, D, generator=g)).to(torch.bfloat16).to(DEV)
    w1 = (torch.randn(2 * F, D, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    w2 = (torch.randn(D, F, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    assert kernels.ffn_stream_supported(x, w1, w2)
    h_ref = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_skinny_swiglu(x, w1, h_ref)
    want = h_ref.double().cpu() @ w2.double().cpu().t()
    gate_up = x.double().cpu() @ w1.double().cpu().t()
    h64 = torch.nn.functional.silu(gate_up[:, :F]) * gate_up[:, F:]
    barrier = torch.zeros(kernels.FFN_SYNC_WORDS, dtype=torch.int32, device=DEV)
    for _ in range(3):
        part = kernels.ffn_stream(x, w1, w2, barrier)
        got = part.sum(0).double().cpu()
        assert torch.isfinite(got).all()
        # h is rounded to bfloat16 between the products in both paths: equal to the two-launch result up to
        # the order of float32 sums, and close to float64 throughout
        assert (got - want).abs().max() <= 1e-4 * want.abs().max() + 1e-6
        assert (got - h64 @ w2.double().cpu().t()).abs().max() <= 2e-2 * want.abs().max()
    assert kernels.gemm_stream_status() == 0


# ---- a wait that runs out: the kernel ends, the status word says so, the host raises
@pytest.mark.gpu
@pytest.mark.parametrize("name", ["gemm_stream", "gemm_tc5", "attention_tc5", "attention_flash"])
def test_a_wait_that_runs_out_ends_the_kernel_and_is_reported_once(name):
    """Each library's own wait function, on an mbarrier nobody arrives at, with a limit of a few thousand
    polls: the launch returns, the library's status word is set, ``check_status`` raises once, and the
    device goes on working."""
    from qwen_decoder_b200 import kernels
    kernels.check_status()                      # clean before
    kernels.wait_probe(name, 4096)
    torch.cuda.synchronize()
    with pytest.raises(kernels.KernelError, match=name):
        kernels.check_status()
    kernels.check_status()                      # reported once
    x = torch.arange(1000, device=DEV, dtype=torch.float32)
    assert float((x * 2).sum()) == 999000.0


@pytest.mark.gpu
def test_a_grid_barrier_that_runs_out_is_reported_and_repaired(tmp_path):
    """The CTAs of the one-launch feed-forward wait for each other's columns of h through counters, with a
    bounded spin.  With a counter that no count of tiles can bring to its target the spin runs out (two
    seconds), the step's results are void, the runner's look at the status raises and puts the words back; the
    steps after it are right again."""
    import plain_model
    from tiny_configs import make_folder
    from qwen_decoder_b200 import kernels
    from qwen_decoder_b200.engine import ModelRunner, StepEntry
    folder = make_folder("D", str(tmp_path))
    cfg, w = plain_model.read_folder(folder)
    runner = ModelRunner.from_folder(folder, dtype="bfloat16", device=DEV, num_pages=8, use_graphs=False)
    seq = [5, 17, 3, 250, 99, 7, 1, 64, 12, 33]
    want = plain_model.forward(cfg, w, seq).numpy()
    rc = runner.open("r")
    runner.step([StepEntry(rc, seq[:7], [6])])
    runner.step([StepEntry(rc, seq[7:8], [0])])
    ff = runner.model.layers[0].feed_forward
    assert ff._barrier is not None, "the decode step did not run the one-launch feed-forward"
    runner.check_status()
    ff._barrier[0] = 1 << 30                    # tiles counted from here never reach the chunk's number
    runner.step([StepEntry(rc, seq[8:9], [0])])
    with pytest.raises(kernels.KernelError, match="gemm_stream"):
        runner.check_status()
    assert ff._barrier.tolist() == [0] * kernels.FFN_SYNC_WORDS
    logits = runner.step([StepEntry(rc, seq[9:10], [0])])
    runner.check_status()
    # position 8 was computed by the void step: its cache entries are suspect, so compare a fresh request
    rc2 = runner.open("again")
    logits = runner.step([StepEntry(rc2, seq, [9])])
    runner.check_status()
    assert float((logits[0].float().cpu() - torch.from_numpy(want[9])).abs().max()) <= 3e-2 * float(np.abs(want).max())


@pytest.mark.gpu
def test_generate_raises_when_a_wait_ran_out(tmp_path):
    """A short generation (far fewer steps than the routine look at the status words) does not hand out
    tokens of a run in which a kernel's wait ran out."""
    from tiny_configs import make_folder
    from qwen_decoder_b200 import kernels
    from qwen_decoder_b200.engine import Engine, SamplingParams
    folder = make_folder("A", str(tmp_path))
    eng = Engine(folder, dtype="bfloat16", device=DEV, num_pages=16)
    assert len(eng.generate([[1, 2, 3]], SamplingParams(max_new_tokens=4, ignore_eos=True))[0]) == 4
    kernels.wait_probe("gemm_stream", 4096)
    with pytest.raises(kernels.KernelError):
        eng.generate([[4, 5, 6]], SamplingParams(max_new_tokens=4, ignore_eos=True))
    kernels.check_status()


def test_guard_regions_catch_a_stray_write(guard_regions):
    """The guard regions themselves: a write one element past a buffer, as an off-by-one index in a kernel would
    make it, changes the margin that the end of every test in this file checks."""
    t = torch.empty(8, 16, dtype=torch.bfloat16, device=DEV)
    raw, nbytes, shape, dtype = guard_regions[-1]
    assert shape == (8, 16) and nbytes == 8 * 16 * 2 and t.data_ptr() == raw.data_ptr() + 1024
    flat = t.view(-1)
    torch.as_strided(flat, (1,), (1,), flat.storage_offset() + flat.numel()).fill_(1.0)
    assert not bool((raw[1024 + nbytes:] == 0xA5).all())
    raw[1024 + nbytes:].fill_(0xA5)                   # put it back: the check at the end of this test must pass
