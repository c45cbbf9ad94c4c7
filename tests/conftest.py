import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def guard_regions(monkeypatch):
    """Guard regions around device memory, for the kernel tests: every CUDA tensor that the test or the code
    under test makes with torch.empty / zeros / full / empty_like lies between two margins of a sentinel
    byte inside one allocation, and at the end of the test every margin must still hold the sentinel.  A
    kernel that writes before or past a buffer it was given -- an output, scratch memory, a cache -- is
    caught even when the stray write spoils no value that the test compares.  (compute-sanitizer is not
    available where these tests run; this stands in for its bounds check on writes.)"""
    import torch
    MARGIN, SENTINEL = 1024, 0xA5
    real = {n: getattr(torch, n) for n in ("empty", "zeros", "full", "empty_like")}
    made = []

    def on_cuda(device):
        return device is not None and torch.device(device).type == "cuda"

    def guarded(shape, dtype, device, fill=None):
        dtype = dtype or torch.get_default_dtype()
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        es = real["empty"]((), dtype=dtype).element_size()
        raw = real["empty"](n * es + 2 * MARGIN, dtype=torch.uint8, device=device)
        raw[:MARGIN].fill_(SENTINEL)
        raw[MARGIN + n * es:].fill_(SENTINEL)
        made.append((raw, n * es, shape, dtype))
        t = raw[MARGIN:MARGIN + n * es].view(dtype).view(shape)
        if fill is not None:
            t.fill_(fill)
        return t

    def shape_of(size):
        return size[0] if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)) else size

    def empty(*size, dtype=None, device=None, **kw):
        if not on_cuda(device) or kw:
            return real["empty"](*size, dtype=dtype, device=device, **kw)
        return guarded(shape_of(size), dtype, device)

    def zeros(*size, dtype=None, device=None, **kw):
        if not on_cuda(device) or kw:
            return real["zeros"](*size, dtype=dtype, device=device, **kw)
        return guarded(shape_of(size), dtype, device, fill=0)

    def full(size, fill_value, dtype=None, device=None, **kw):
        if not on_cuda(device) or kw:
            return real["full"](size, fill_value, dtype=dtype, device=device, **kw)
        if dtype is None:
            dtype = torch.get_default_dtype() if isinstance(fill_value, float) else torch.int64
        return guarded(size, dtype, device, fill=fill_value)

    def empty_like(t, **kw):
        if not t.is_cuda or kw or not t.is_contiguous():
            return real["empty_like"](t, **kw)
        return guarded(t.shape, t.dtype, t.device)

    for name, fn in (("empty", empty), ("zeros", zeros), ("full", full), ("empty_like", empty_like)):
        monkeypatch.setattr(torch, name, fn)
    yield made
    for name, fn in real.items():
        monkeypatch.setattr(torch, name, fn)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    for raw, nbytes, shape, dtype in made:
        before, after = raw[:MARGIN], raw[MARGIN + nbytes:]
        assert bool((before == SENTINEL).all()), f"a kernel wrote BEFORE a {dtype} buffer of shape {shape}"
        assert bool((after == SENTINEL).all()), f"a kernel wrote PAST a {dtype} buffer of shape {shape}"
    made.clear()
