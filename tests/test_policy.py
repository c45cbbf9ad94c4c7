"""The product policies that need no GPU: which library products are given as a batch over shares of K, and which
products of 9 to 16 tokens keep their tokens resident in the streamer."""
import pytest

from qwen_decoder_b200 import kernels
from qwen_decoder_b200.parts import matmul_backend


@pytest.mark.parametrize("T,N,K,want", [
    (16, 2048, 11008, 0),        # up to 16 tokens the few-token kernels take the product
    (17, 2048, 11008, 4), (64, 2048, 11008, 4), (256, 2048, 11008, 4),
    (257, 2048, 11008, 0), (576, 2048, 11008, 0),       # above 256 tokens the plain product stands
    (64, 3584, 18944, 4), (384, 3584, 18944, 0),
    (64, 5120, 27648, 0),        # too many output features to leave the GPU idle
    (64, 2048, 2048, 0),         # K no longer than the output is wide
    (64, 2560, 2048, 0),
    (64, 520, 4104, 0),          # shares of 1,026 columns would not start on 16-byte boundaries
    (300, 136, 4128, 0), (200, 136, 4112, 0), (200, 136, 4128, 4),
])
def test_library_shares(T, N, K, want, monkeypatch):
    assert matmul_backend.mode == "auto"
    assert matmul_backend.library_shares(T, N, K) == 0          # off unless a number of shares is set
    monkeypatch.setattr(matmul_backend, "library_split_k", 4)
    assert matmul_backend.library_shares(T, N, K) == want


def test_library_shares_follow_the_mode(monkeypatch):
    monkeypatch.setattr(matmul_backend, "library_split_k", 4)
    assert matmul_backend.library_shares(64, 2048, 11008) == 4
    monkeypatch.setattr(matmul_backend, "mode", "cublas")
    assert matmul_backend.library_shares(64, 2048, 11008) == 0
    monkeypatch.setattr(matmul_backend, "mode", "auto")
    monkeypatch.setattr(matmul_backend, "library_split_k", 0)
    assert matmul_backend.library_shares(64, 2048, 11008) == 0


@pytest.mark.parametrize("T,K,want", [
    (8, 2048, 0), (9, 2048, 2), (16, 2048, 2), (17, 2048, 0),
    (12, 11008, 11), (16, 1000, 1), (16, 1032, 2), (16, 18944, 19), (16, 27648, 27),
    (16, 32768, 32), (16, 32776, 0),          # more shares than the partial sums are allowed to have
])
def test_stream_resident_shares(T, K, want):
    assert kernels.skinny_impl == "stream"
    assert kernels.stream_resident_shares(T, K) == want


def test_stream_resident_shares_follow_the_limits(monkeypatch):
    monkeypatch.setattr(kernels, "STREAM_RESIDENT_TOKENS", 8)
    assert kernels.stream_resident_shares(12, 2048) == 0
    monkeypatch.setattr(kernels, "STREAM_RESIDENT_TOKENS", 16)
    monkeypatch.setattr(kernels, "skinny_impl", "regs")
    assert kernels.stream_resident_shares(12, 2048) == 0
