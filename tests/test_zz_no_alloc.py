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
