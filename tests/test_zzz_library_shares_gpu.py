"""The library product over shares of K (``parts/matmul_backend.py``: ``library_split_k``, off by default), through the
Linear part and through the native prompt loop.  These run after every other test file: with the batched product on,
later prompt steps of the same process have shown a wrong row tile now and then, for a reason that was not found."""
import random

import numpy as np
import pytest
import torch

import plain_model
from tiny_configs import TINY
from test_native_prompt_gpu import run_portions, runner_for
from test_parts_gpu import DEV, bind, close, total

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,N,K", [(17, 136, 4096), (40, 2048, 4128), (64, 520, 11008), (64, 136, 4104), (256, 136, 4128),
                                   (300, 136, 4128)])
def test_linear_part_as_partial_sums_of_a_batched_library_product(T, N, K, monkeypatch):
    """17 to 256 tokens, a long K and few output features: four shares of K as one batched product; a K that does
    not divide into shares of whole 16-byte pieces, and more tokens, take the plain product."""
    from qwen_decoder_b200.parts.linear import Linear
    from qwen_decoder_b200.parts import matmul_backend
    monkeypatch.setattr(matmul_backend, "library_split_k", 4)       # off by default
    lin = Linear(K, [("p", N)], bias=False)
    w = bind(lin, torch.bfloat16, 8, scale=0.03)
    x = torch.randn(T, K, generator=torch.Generator().manual_seed(9))
    x[:, K // 2:] *= 3.0                       # the shares of K differ in weight
    x = x.to(torch.bfloat16)
    got = lin.forward_partial(x.to(DEV))
    shares = matmul_backend.library_shares(T, N, K)
    assert shares == (0 if T > 256 or K % 32 else 4)
    assert (got.dim() == 3 and got.shape[0] == shares and got.dtype == torch.float32) if shares else got.dim() == 2
    close(total(got), plain_model.linear(x.double(), w["p.weight"]), torch.bfloat16)


def test_native_prompt_with_the_down_projection_in_shares(tmp_path, monkeypatch):
    """An intermediate size of 4,128 with a hidden size of 96: the native loop gives the down projection to the
    library as a batch over four shares of K up to 256 tokens (the plain product above) and the next norm adds the
    float32 partial sums -- also the final norm, which gathers rows."""
    from qwen_decoder_b200.config import Qwen2Config
    from qwen_decoder_b200.weights import write_random_model
    from qwen_decoder_b200.parts import matmul_backend
    monkeypatch.setattr(matmul_backend, "library_split_k", 4)       # off by default
    cfg_dict = dict(TINY["D"], intermediate_size=4128, max_position_embeddings=1024)
    assert matmul_backend.library_shares(70, 96, 4128) == 4 and matmul_backend.library_shares(300, 96, 4128) == 0
    folder = write_random_model(Qwen2Config.from_dict(cfg_dict), str(tmp_path), 17, dtype=torch.bfloat16)
    cfg, w = plain_model.read_folder(folder)
    rng = random.Random(12)
    seqs = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (420, 97, 40)]
    cuts = [70, 300, 50]
    native, parts = runner_for(folder, True), runner_for(folder, False)
    a = run_portions(native, seqs, cuts)
    b = run_portions(parts, seqs, cuts)
    assert native.model.native_prompt.steps == 3
    want = [plain_model.forward(cfg, w, s).numpy() for s in seqs]
    scale = max(float(np.abs(x).max()) for x in want)
    assert a.keys() == b.keys() and len(a) == 6
    for (i, pos), row in a.items():
        assert np.isfinite(row).all()
        assert np.abs(row - b[(i, pos)]).max() <= 2e-2 * scale
        assert np.abs(row - want[i][pos]).max() <= 3e-2 * scale
    native.cache.check()
