"""Reading and writing the safetensors container.

Layout of a file: an 8-byte little-endian header length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the raw little-endian tensor data; offsets are relative to the end of the
header.  This stands where the reference parses GGUF (gguf_loader.cpp:107-156)
and maps the file (common.cpp:16-35): tensors are views into one memory map and
are copied only when they go to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Mapping, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One mapped safetensors file; ``tensor(name)`` returns a CPU view."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file too short ({size} bytes) to hold a safetensors header")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds file size {size} (truncated file?)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        data_len = size - self._data_start
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for tensor {name!r}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=_DTYPES[dt]).element_size()
            if e - b != want:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {list(shape)} {dt} needs {want} bytes, "
                    f"header gives {e - b}")
            if b < 0 or e > data_len:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} lies at bytes [{b}, {e}) but the file holds only "
                    f"{data_len} data bytes (truncated file?)")
            self._entries[name] = (_DTYPES[dt], shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self):
        return list(self._entries)

    def info(self, name: str):
        dt, shape, _, _ = self._entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, e = self._entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        numel = 1
        for s in shape:
            numel *= s
        t = torch.frombuffer(self._mm, dtype=dt, count=numel, offset=self._data_start + b)
        return t.reshape(shape)


def open_model_tensors(model_dir: str) -> Dict[str, Tuple[SafetensorsFile, str]]:
    """Map every tensor name in a model folder to the file that holds it.

    Accepts ``model.safetensors`` or ``model.safetensors.index.json`` with shards.
    """
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    out: Dict[str, Tuple[SafetensorsFile, str]] = {}
    if os.path.isfile(single):
        f = SafetensorsFile(single)
        for n in f.names():
            out[n] = (f, n)
        return out
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as fh:
            wm = json.load(fh).get("weight_map", {})
        files: Dict[str, SafetensorsFile] = {}
        for name, fname in wm.items():
            if fname not in files:
                files[fname] = SafetensorsFile(os.path.join(model_dir, fname))
            if name not in files[fname]._entries:
                raise SafetensorsError(f"{index}: tensor {name!r} is not in shard {fname!r}")
            out[name] = (files[fname], name)
        return out
    raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in {model_dir!r}")


def save_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write ``tensors`` (any device; written from CPU copies) as one safetensors file."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
