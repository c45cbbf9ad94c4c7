"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.  The reference has no such mode (it needs a GGUF file,
gpu_decoder.cu:169-188); tests and benchmarks here run without any checkpoint.

Every tensor has its own generator seeded from (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or in which order they are made.
"""
from __future__ import annotations

import hashlib
import os
from typing import Dict, Iterable

import torch

from ..config import describe_model, write_config_json
from .loader import TensorSpec
from .safetensors_io import save_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(spec: TensorSpec, seed: int, dtype=torch.bfloat16, device="cpu",
                  std: float = 0.02, norm_std: float = 0.1) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    if spec.init == "around_one":
        t.normal_(0.0, norm_std, generator=g).add_(1.0)
    else:
        t.normal_(0.0, std, generator=g)
    return t.to(dtype)


def random_tensors(specs: Iterable[TensorSpec], seed: int, dtype=torch.bfloat16, device="cpu",
                   std: float = 0.02, norm_std: float = 0.1) -> Dict[str, torch.Tensor]:
    return {s.name: random_tensor(s, seed, dtype, device, std, norm_std) for s in specs}


def write_random_model(config, model_dir: str, seed: int, dtype=torch.bfloat16,
                       std: float = 0.02, norm_std: float = 0.1) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config``; returns the folder."""
    from ..parts.model import build_model  # parts import weights.loader; avoid a cycle at import
    model = build_model(describe_model(config))
    os.makedirs(model_dir, exist_ok=True)
    write_config_json(config, model_dir)
    tensors = random_tensors(model.tensor_specs(), seed, dtype, "cpu", std, norm_std)
    save_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                     {"format": "pt", "seed": str(seed)})
    return model_dir
