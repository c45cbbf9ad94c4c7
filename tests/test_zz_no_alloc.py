"""The allocation-free decode attention entry point (csrc/decode_attention_noalloc.h).

It is meant for callers that cannot allocate device memory -- code inside a stream capture or a
latency-critical loop, plug-ins whose host owns all device memory, processes under a memory budget
fixed before this library was loaded.  The test calls the entry point through its exported C symbol,
the way such a caller would, twice in a row with different inputs (the second call finds the first
call's leftovers in the shared scratch array), and checks each result against the ordinary entry
point, which takes its scratch from the caller.  It also checks that the second call does not change
the amount of free device memory and that a call beyond the fixed maximum is refused with a clear
message.  The file name makes pytest collect it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup(seed, lens, H, G, d, page_size):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + page_size - 1) // page_size for n in lens) + 2
    kv = torch.randn(n_pages, 2, G, page_size, d, generator=g).to(torch.bfloat16)
    perm = torch.randperm(n_pages, generator=g).tolist()
    mb = max((n + page_size - 1) // page_size for n in lens)
    bt = torch.full((len(lens), mb), -1, dtype=torch.int32)
    for i, n in enumerate(lens):
        for p in range((n + page_size - 1) // page_size):
            bt[i, p] = perm.pop()
    q = torch.randn(len(lens), H * d, generator=g).to(torch.bfloat16)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    tr = torch.arange(len(lens), dtype=torch.int32)
    return [t.to(DEV) for t in (q, kv, bt, tr, pos)]


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from qwen_decoder_b200 import kernels
    from qwen_decoder_b200.csrc.build import library
    lib = library("decode_attention_noalloc")
    fn = lib.qd_decode_attention_noalloc
    fn.restype = ctypes.c_int
    lib.qd_decode_attention_noalloc_strerror.restype = ctypes.c_char_p
    lib.qd_decode_attention_noalloc_scratch_floats.restype = ctypes.c_longlong
    H, G, d, page_size, splits = 16, 2, 128, 16, 6
    scale = 1.0 / math.sqrt(d)
    P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

    def call(q, kv, bt, tr, pos, out, n_splits):
        T = q.shape[0]
        return fn(P(q.data_ptr()), LL(q.stride(0)), P(out.data_ptr()), P(kv.data_ptr()), P(bt.data_ptr()),
                  I(bt.shape[1]), P(tr.data_ptr()), P(pos.data_ptr()), I(T), I(H), I(G), I(d), I(page_size),
                  F(scale), I(0), I(n_splits), P(torch.cuda.current_stream().cuda_stream))

    free_after_first = None
    for seed, lens in ((31, [700, 33, 1, 256, 1025]), (32, [90, 1500, 17])):
        q, kv, bt, tr, pos = _setup(seed, lens, H, G, d, page_size)
        T = len(lens)
        want = torch.empty(T, H * d, dtype=torch.bfloat16, device=DEV)
        kernels.decode_attention(q, q.stride(0), want, kv, bt, tr, pos, T, H, G, d, page_size, scale, 0, splits)
        got = torch.full((T, H * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        torch.cuda.synchronize()
        if free_after_first is not None:
            free_before = torch.cuda.mem_get_info()[0]
        rc = call(q, kv, bt, tr, pos, got, splits)
        torch.cuda.synchronize()
        assert rc == 0, lib.qd_decode_attention_noalloc_strerror(rc)
        if free_after_first is not None:
            assert torch.cuda.mem_get_info()[0] == free_before        # the call took no device memory
        free_after_first = torch.cuda.mem_get_info()[0]
        err = float((got.float() - want.float()).abs().max())
        assert err <= 1e-2 * float(want.float().abs().max()), err      # the tolerance of the kernel tests
        assert not torch.isnan(got.float()).any()
        # one CTA per (request, kv head): no scratch at all, same answer
        got1 = torch.empty_like(got)
        assert call(q, kv, bt, tr, pos, got1, 1) == 0
        torch.cuda.synchronize()
        assert float((got1.float() - want.float()).abs().max()) <= 1e-2 * float(want.float().abs().max())

    # beyond the fixed maximum: refused before anything is launched, with a message that says why
    q, kv, bt, tr, pos = _setup(33, [40] * 8, H, G, d, page_size)
    need = lib.qd_decode_attention_noalloc_scratch_floats(I(8), I(H), I(d), I(1000))
    assert need == 8 * H * 1000 * (d + 2) > 2 * 1024 * 1024
    out = torch.zeros(8, H * d, dtype=torch.bfloat16, device=DEV)
    rc = call(q, kv, bt, tr, pos, out, 1000)
    torch.cuda.synchronize()
    assert rc == 20001 and float(out.float().abs().max()) == 0.0
    assert b"more scratch than" in lib.qd_decode_attention_noalloc_strerror(rc)
    # sizes the kernel does not take are refused too (head size 100)
    rc = fn(P(q.data_ptr()), LL(q.stride(0)), P(out.data_ptr()), P(kv.data_ptr()), P(bt.data_ptr()), I(bt.shape[1]),
            P(tr.data_ptr()), P(pos.data_ptr()), I(8), I(H), I(G), I(100), I(page_size), F(scale), I(0), I(2),
            P(torch.cuda.current_stream().cuda_stream))
    assert rc == 20002


def test_no_alloc_entry_point_against_the_plain_formulas_at_the_edges():
    """The second kernel of this entry point (the one that adds the shares up, where the ordinary entry point
    lets the last CTA do it) with what makes shares uneven or empty: a window whose first visible key lies inside
    a 16-key chunk, pages before the window given back (-1 in the block table), more shares than the shortest
    request has chunks.  Compared with the plain formulas, not with the other entry point."""
    import plain_model
    from qwen_decoder_b200.csrc.build import library
    lib = library("decode_attention_noalloc")
    fn = lib.qd_decode_attention_noalloc
    fn.restype = ctypes.c_int
    lib.qd_decode_attention_noalloc_strerror.restype = ctypes.c_char_p
    H, G, d, page_size, window = 6, 2, 64, 16, 75
    scale = 1.0 / math.sqrt(d)
    P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lens = [300, 20, 76, 131, 1]                    # keys lens[i] - window .. lens[i] - 1 are visible
    g = torch.Generator().manual_seed(41)
    ks = [torch.randn(n, G, d, generator=g).to(torch.bfloat16) for n in lens]
    vs = [torch.randn(n, G, d, generator=g).to(torch.bfloat16) for n in lens]
    n_pages = sum((n + page_size - 1) // page_size for n in lens) + 1
    kv = torch.zeros(n_pages, 2, G, page_size, d, dtype=torch.bfloat16)
    mb = max((n + page_size - 1) // page_size for n in lens)
    bt = torch.full((len(lens), mb), -1, dtype=torch.int32)
    page = 0
    for i, n in enumerate(lens):
        first_needed = max(0, n - window) // page_size      # pages below it were given back when the window passed
        for lp in range((n + page_size - 1) // page_size):
            if lp < first_needed:
                continue
            bt[i, lp] = page
            lo, hi = lp * page_size, min(n, (lp + 1) * page_size)
            kv[page, 0, :, :hi - lo, :] = ks[i][lo:hi].transpose(0, 1)
            kv[page, 1, :, :hi - lo, :] = vs[i][lo:hi].transpose(0, 1)
            page += 1
    q = torch.randn(len(lens), H * d, generator=g).to(torch.bfloat16)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    tr = torch.arange(len(lens), dtype=torch.int32)
    want = []
    for i, n in enumerate(lens):
        qq = torch.zeros(n, H * d, dtype=torch.float64)
        qq[n - 1] = q[i].double()
        want.append(plain_model.attention(qq, ks[i].double().reshape(n, G * d), vs[i].double().reshape(n, G * d),
                                          H, G, d, window)[n - 1])
    want = torch.stack(want)
    dq, dkv, dbt, dtr, dpos = (t.to(DEV) for t in (q, kv, bt, tr, pos))
    for splits in (1, 3, 7, 24):                    # 24 shares: more than any of these requests has chunks in its window
        got = torch.full((len(lens), H * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        rc = fn(P(dq.data_ptr()), LL(dq.stride(0)), P(got.data_ptr()), P(dkv.data_ptr()), P(dbt.data_ptr()),
                I(dbt.shape[1]), P(dtr.data_ptr()), P(dpos.data_ptr()), I(len(lens)), I(H), I(G), I(d), I(page_size),
                F(scale), I(window), I(splits), P(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert rc == 0, lib.qd_decode_attention_noalloc_strerror(rc)
        err = float((got.double().cpu() - want).abs().max())
        assert err <= 1e-2 * float(max(v.abs().max() for v in vs)), (splits, err)
