"""Binding tensors to a model by name.

The reference looks each tensor up by name with a linear search and returns a null
pointer on a miss, which crashes later in the upload (common.cpp:94-102,
gpu_decoder.cu:15-61); shapes and dtypes are never checked (common.cpp:104-112).
Here every tensor the model declares is checked against the folder first, and all
faults come out in one error: missing names, unexpected names, wrong shapes.

Storage rule: a tensor is kept as it is stored if that is bfloat16, float16 or a
32-bit type (float16 is the reference's own weight format, decoded exactly by its
float32 forward, common.cpp:104-112, cpu_decoder.cpp:55-62: a part that computes in
float32 gets every stored bit, one that computes in bfloat16 rounds once);
float64 becomes float32; integer tables become int32.  What precision a part
computes in is the part's business (``bind``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from .safetensors_io import open_model_tensors


class WeightError(ValueError):
    """Missing, unexpected or mis-shaped tensors; ``missing``/``unexpected``/``wrong_shape`` list them."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part needs: full name, shape, and how random weights fill it
    (``normal``: N(0, std); ``around_one``: 1 + N(0, norm_std), for norm scales)."""
    name: str
    shape: Tuple[int, ...]
    init: str = "normal"


def storage_dtype(dt: torch.dtype) -> torch.dtype:
    """The dtype a loaded tensor is kept in (see the module's storage rule)."""
    if dt in (torch.bfloat16, torch.float16, torch.float32, torch.int32):
        return dt
    if dt == torch.float64:
        return torch.float32
    if dt in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    raise WeightError(f"unsupported tensor dtype {dt}")


def check_tensors(specs: Iterable[TensorSpec], found: Mapping[str, Tuple[int, ...]], where: str = "",
                  ignorable: Iterable[str] = ()) -> None:
    """Raise one ``WeightError`` that lists every fault, or return.  Tensors named in ``ignorable`` may be
    present without being used (a warning says so): a model with tied embeddings whose file still
    carries an output matrix."""
    want = {}
    for s in specs:
        want[s.name] = tuple(s.shape)
    missing = sorted(n for n in want if n not in found)
    ignorable = set(ignorable)
    ignored = sorted(n for n in found if n not in want and n in ignorable)
    if ignored:
        import warnings
        warnings.warn(f"weights{' in ' + where if where else ''}: tensors present but not used by this "
                      f"configuration: {', '.join(ignored)}")
    unexpected = sorted(n for n in found if n not in want and n not in ignorable)
    wrong = sorted((n, want[n], tuple(found[n])) for n in want if n in found and tuple(found[n]) != want[n])
    if not (missing or unexpected or wrong):
        return
    lines = [f"weights{' in ' + where if where else ''} do not fit the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(
            f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in wrong))
    raise WeightError("\n".join(lines), missing, unexpected, wrong)


class TensorSource:
    """Named tensors for ``bind``: fetched one at a time so that a large model is
    never held twice.  ``get(name)`` returns the tensor in its storage dtype."""

    def __init__(self, fetch, shapes: Dict[str, Tuple[int, ...]], where: str = ""):
        self._fetch = fetch
        self.shapes = shapes
        self.where = where

    def get(self, name: str) -> torch.Tensor:
        t = self._fetch(name)
        return t.to(storage_dtype(t.dtype))

    @classmethod
    def from_folder(cls, model_dir: str) -> "TensorSource":
        entries = open_model_tensors(model_dir)
        shapes = {n: f.info(k)[1] for n, (f, k) in entries.items()}
        for n, (f, k) in entries.items():
            storage_dtype(f.info(k)[0])  # unsupported dtypes fail here, with the name below
        return cls(lambda n: entries[n][0].tensor(entries[n][1]), shapes, model_dir)

    @classmethod
    def from_dict(cls, tensors: Mapping[str, torch.Tensor], where: str = "memory") -> "TensorSource":
        return cls(lambda n: tensors[n], {n: tuple(t.shape) for n, t in tensors.items()}, where)


def load_into(model, source: TensorSource, dtype: torch.dtype, device) -> None:
    """Check ``source`` against ``model.tensor_specs()`` and bind every part."""
    check_tensors(model.tensor_specs(), source.shapes, source.where,
                  getattr(model, "ignorable_tensors", lambda: ())())
    model.bind(source, dtype, torch.device(device))
